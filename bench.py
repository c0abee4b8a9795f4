"""Decode and prefill throughput of the engine on one B200, as one JSON line.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]

The default run builds the headline model (28 layers, hidden 2048, 16/8 heads
of 128, intermediate 6144, vocabulary 151936, tied head) with random bfloat16 weights,
holds 8 requests whose contexts end at 4096 tokens, and times K decode steps.
`value` is decoded tokens per second timed on the device; `e2e` is the same measured
through the Python entry point's generation loop, which copies every step's inputs
from pinned host memory and reads the chosen tokens back. `prefill` is one step of
2,048 prompt tokens; `roofline` relates the decode step's time to the bytes it must
read (every weight once, and the live requests' cache). `points` holds decode at
batch 1 and 64, two mixed steps (milliseconds a step: eight decoding requests at
4,096 tokens beside a 256-token portion of a prompt, and a lone 128-token portion) and the
time to read a prompt of 8,192 tokens in portions of 512 (a token budget).
`kernels` times each class of kernel alone (operands rotated through more memory than
L2 holds, replayed from a CUDA graph) against the measured peaks: the streamed product
of a decode step, the head, decode attention (GB/s), the prefill product and prefill
attention (TFLOP/s). Data is synthetic: seeded uniform-random token ids.

`--only fokalorn` is a record of its own: prefill and decode throughput of the Fokalorn design at a
few sizes that resemble a real model's layers (random weights), beside Muse-Glimmer at equal width,
depth, heads and feed-forward, and each kernel of the new design alone against its roofline beside
the like kernel of Muse-Glimmer (`--size` picks one size). `--only dolutar` is the same kind of record for
the Dolutar design (sliding-window attention with kept first positions and a sink, a clamped gated unit,
routed experts), beside Muse-Glimmer with sliding attention at equal width, depth, heads, window and
active feed-forward width. `--only bobarax` is that record for the Bobarax design (decayed linear attention,
run-masked attention with capped scores, gated windowed attention, experts chosen by a table), beside Dolutar
at equal width, depth, heads, window and experts; its kernels stand beside the like kernels of Dolutar and,
for the recurrence, of Fokalorn. `--only narezen` is that record for the Narezen design (attention beside a
decayed linear-attention state in one mixer, a gated recurrence over channels, sigmoid-routed experts weighted
on their inputs with a shared expert), beside Bobarax at equal width, depth, heads and experts; its kernels
stand beside the like kernels of Bobarax.
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
sys.path.insert(0, str(ROOT))

CONFIG2 = {
    "architectures": ["MuseGlimmerForConditionalGeneration"], "model_type": "muse_glimmer",
    "text_config": {
        "hidden_size": 2048, "intermediate_size": 6144, "num_hidden_layers": 28, "num_attention_heads": 16,
        "num_key_value_heads": 8, "head_dim": 128, "vocab_size": 151936, "rms_norm_eps": 1e-6, "post_norm_eps": 1e-6,
        "sliding_window": 4096, "qk_scale_factor": 1.0, "output_multiplier": 1.0, "final_logit_softcapping": 30.0,
        "layer_types": ["full_attention"] * 28, "layer_rope_theta": [1000000.0] * 28,
        "rope_parameters": {"rope_theta": 1000000.0, "rope_type": "default"}, "eos_token_id": [],
        "tie_word_embeddings": True,
    },
}
CONFIG3 = {
    "architectures": ["MuseGlimmerForConditionalGeneration"], "model_type": "muse_glimmer",
    "text_config": {
        "hidden_size": 4096, "intermediate_size": 12288, "num_hidden_layers": 36, "num_attention_heads": 32,
        "num_key_value_heads": 8, "head_dim": 128, "vocab_size": 151936, "rms_norm_eps": 1e-6, "post_norm_eps": 1e-6,
        "sliding_window": 8192, "qk_scale_factor": 1.0, "output_multiplier": 1.0, "final_logit_softcapping": 30.0,
        "layer_types": ["full_attention"] * 36, "layer_rope_theta": [1000000.0] * 36,
        "rope_parameters": {"rope_theta": 1000000.0, "rope_type": "default"}, "eos_token_id": [],
        "tie_word_embeddings": False,
    },
}
CONFIGS = {2: (CONFIG2, 4096), 3: (CONFIG3, 8192)}  # the sizes and the context of a benchmark configuration
SEED = 2
CONTEXT = 4096
PREFILL_TOKENS = 2048
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}


def peaks() -> tuple[dict, str]:
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        try:
            data = json.loads(path.read_text())
            flat = {}
            for key in FALLBACK_PEAKS:
                value = data.get(key)
                if isinstance(value, dict):
                    value = value.get("value")
                flat[key] = float(value) if value else FALLBACK_PEAKS[key]
            return flat, "measured"
        except (ValueError, TypeError):
            pass
    return dict(FALLBACK_PEAKS), "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while a region runs."""

    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self) -> None:
        self.rows: list[list[str]] = []
        self.process = None

    def __enter__(self):
        try:
            self.process = subprocess.Popen(
                ["nvidia-smi", "-i", "0", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "100"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.process = None
        return self

    def _read(self) -> None:
        for line in self.process.stdout:
            self.rows.append([cell.strip() for cell in line.split(",")])

    def __exit__(self, *exc) -> None:
        if self.process is not None:
            self.process.terminate()
            self.thread.join(timeout=2)

    def summary(self) -> dict:
        clocks = [int(r[0]) for r in self.rows if r and r[0].isdigit()]
        peak = [int(r[1]) for r in self.rows if len(r) > 1 and r[1].isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(len(r) > i + 2 and r[i + 2] == "Active" for r in self.rows)]
        return {"sm_mhz": statistics.median(clocks) if clocks else None, "sm_max_mhz": max(peak) if peak else None,
                "reasons": reasons, "samples": len(clocks)}


def model_bytes(text: dict, layers: int) -> tuple[int, int, int]:
    """(weight bytes a decode step reads, cache bytes per token of context, parameters)."""
    h, i, d = text["hidden_size"], text["intermediate_size"], text["head_dim"]
    q, kv = text["num_attention_heads"] * d, text["num_key_value_heads"] * d
    per_layer = h * (2 * q + 2 * kv) + q * h + 3 * h * i
    head = text["vocab_size"] * h
    params = layers * per_layer + head * (1 if text["tie_word_embeddings"] else 2)
    return 2 * (layers * per_layer + head), 2 * 2 * layers * kv, params


def run(args) -> dict:
    import torch

    from mlx_omnia_b200.engine.decode_graph import capturing
    from mlx_omnia_b200.engine.engine import Engine, EngineArgs
    from mlx_omnia_b200.engine.generate import Generator
    from mlx_omnia_b200.engine.step import StepEntry
    from mlx_omnia_b200.kernels import ops
    from mlx_omnia_b200.sampling import GenerationOptions

    raw = json.loads(json.dumps(CONFIGS[args.config][0]))
    text = raw["text_config"]
    full_layers = text["num_hidden_layers"]
    layers = args.layers or full_layers
    text["num_hidden_layers"] = layers
    text["layer_types"], text["layer_rope_theta"] = text["layer_types"][:layers], text["layer_rope_theta"][:layers]
    vocab = text["vocab_size"]
    measured, peak_source = peaks()
    weight_bytes, kv_per_token, params = model_bytes(text, layers)

    batches = sorted({1, args.batch, 64}) if args.only == "all" else [args.batch]
    cache_tokens = max(batches) * (args.context + 16) + max(PREFILL_TOKENS, args.prefill_tokens,
                                                              32768 + 16 if args.only == "portions" else 8192 + 16,
                                                              (max(args.steps, 8) + max(args.warmup, 3) + 2) * args.portion)
    cache_tokens = max(cache_tokens, args.pool_tokens)
    engine = Engine.from_random(raw, SEED, EngineArgs(dtype="bfloat16", page_size=16, cache_tokens=cache_tokens,
                                                      max_requests=max(batches) + 1))
    g = torch.Generator().manual_seed(SEED)

    def prompts(count: int, length: int) -> list[list[int]]:
        return torch.randint(0, vocab, (count, length), generator=g).tolist()

    def events():
        return torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)

    def decode(batch: int, steps: int, warmup: int) -> dict:
        """Fill `batch` requests so that the timed steps end at CONTEXT tokens, then time them."""
        total = warmup + steps
        length = args.context - total - 1
        # One step reads all prompts whole, so every request decodes in lockstep afterwards.
        generator = Generator(engine, max_tokens_per_step=batch * length)
        options = GenerationOptions(max_tokens=total + 1, stop=())
        for p in prompts(batch, length):
            generator.add(p, options)
        assert len(generator.step()) == batch
        for _ in range(warmup):
            generator.step()
        torch.cuda.synchronize()
        start, stop = events()
        launches = ops.launches
        wall = time.perf_counter()
        start.record()
        for _ in range(steps):
            outputs = generator.step()
        stop.record()
        torch.cuda.synchronize()
        wall = time.perf_counter() - wall
        ms = start.elapsed_time(stop) / steps
        assert len(outputs) == batch
        context = generator.scheduler.running[0].computed if generator.scheduler.running else args.context
        generator.run()
        return {"ms": ms, "tokens_per_s": batch * 1000.0 / ms, "wall_tokens_per_s": batch * steps / wall,
                "launches": (ops.launches - launches) // steps, "context": context}

    def prefill(tokens: int, steps: int, warmup: int) -> dict:
        times = []
        for index in range(warmup + steps):
            request = engine.cache.open(f"prefill-{index}")
            ids = prompts(1, tokens)[0]
            torch.cuda.synchronize()
            start, stop = events()
            start.record()
            engine.runner.run([StepEntry(request, ids, [tokens - 1])])
            stop.record()
            torch.cuda.synchronize()
            engine.cache.close(request.request_id)
            if index >= warmup:
                times.append(start.elapsed_time(stop))
        ms = statistics.median(times)
        h, d, nq = text["hidden_size"], text["head_dim"], text["num_attention_heads"]
        matmul = 2 * (weight_bytes // 2 - vocab * h) * tokens + 2 * vocab * h  # the head runs on one row
        attention = layers * 4 * nq * d * tokens * (tokens + 1) // 2
        flops = matmul + attention
        return {"value": tokens * 1000.0 / ms, "tokens": tokens, "ms": ms,
                "frac": flops / (ms / 1000.0) / (measured["bf16_tflops"] * 1e12), "flops": flops}

    def mixed(decoders: int, portion: int, steps: int, warmup: int) -> dict:
        """`decoders` requests at `args.context` tokens decode beside `portion` tokens of a long prompt."""
        requests = [engine.cache.open(f"mixed-{i}") for i in range(decoders)]
        reader = engine.cache.open("mixed-reader")
        if decoders:
            engine.runner.run([StepEntry(r, p, []) for r, p in zip(requests, prompts(decoders, args.context - steps - warmup - 1))])
        times, walls = [], []
        for index in range(warmup + steps):
            entries = [StepEntry(r, [1 + index], [0]) for r in requests] + [StepEntry(reader, prompts(1, portion)[0], [])]
            torch.cuda.synchronize()
            start, stop = events()
            wall = time.perf_counter()
            start.record()
            engine.runner.run(entries)
            stop.record()
            torch.cuda.synchronize()
            wall = time.perf_counter() - wall
            if index >= warmup:
                times.append(start.elapsed_time(stop))
                walls.append(wall * 1e3)
        for r in requests + [reader]:
            engine.cache.close(r.request_id)
        return {"ms": statistics.median(times), "wall_ms": statistics.median(walls)}

    def portions(total: int, portion: int) -> float:
        """Milliseconds to read a prompt of `total` tokens in portions of `portion` (a token budget), warm:
        the best of four prompts (steps whose shape has come three times run from captured graphs)."""
        best = None
        for attempt in range(4):
            request = engine.cache.open(f"portions-{attempt}")
            ids = prompts(1, total)[0]
            torch.cuda.synchronize()
            start, stop = events()
            start.record()
            for at in range(0, total, portion):
                engine.runner.run([StepEntry(request, ids[at:at + portion], [portion - 1] if at + portion >= total else [])])
            stop.record()
            torch.cuda.synchronize()
            engine.cache.close(request.request_id)
            best = start.elapsed_time(stop) if best is None else min(best, start.elapsed_time(stop))
        return best

    def kernel_classes() -> dict:
        """Each class of kernel alone, replayed from a graph over operands that do not fit L2."""
        from mlx_omnia_b200.parts.base import KVView, StepContext

        device = engine.runtime.device
        h, inner, d = text["hidden_size"], text["intermediate_size"], text["head_dim"]
        nq, nkv = text["num_attention_heads"], text["num_key_value_heads"]
        draw = lambda *shape: torch.randn(*shape, device=device, dtype=torch.bfloat16) * 0.05

        def timed(body, sets: int) -> float:
            """Seconds per call of `body(i)`, i cycling through `sets` operand sets."""
            side = torch.cuda.Stream()
            with torch.cuda.stream(side):
                for i in range(sets):
                    body(i)
                torch.cuda.synchronize()
                graph = torch.cuda.CUDAGraph()
                with capturing(graph, stream=side):
                    for i in range(sets):
                        body(i)
            torch.cuda.synchronize()
            for _ in range(3):
                graph.replay()
            start, stop = events()
            start.record()
            for _ in range(5):
                graph.replay()
            stop.record()
            torch.cuda.synchronize()
            return start.elapsed_time(stop) / 1e3 / (5 * sets)

        def record(seconds: float, amount: float, peak: float, unit: str) -> dict:
            achieved = amount / seconds / (1e9 if unit == "GB/s" else 1e12)
            return {"achieved": round(achieved, 1), "unit": unit, "frac": round(achieved / peak, 3), "us": round(seconds * 1e6, 2)}

        out = {}
        hbm, tensor = measured["hbm_gbs"], measured["bf16_tflops"]
        # K3: the streamed product of a decode step (gate|up with SwiGLU, 8 rows).
        weights = [draw(2 * inner, h) for _ in range(6)]
        rows8 = draw(8, h)
        out["k3_streamed_product"] = record(timed(lambda i: ops.linear_swiglu(rows8, weights[i]), 6), 2 * 2 * inner * h, hbm, "GB/s")
        # K10: the head with its soft cap, 8 rows.
        table = engine.model.embedding.weight
        out["k10_head"] = record(timed(lambda i: ops.linear_softcap(rows8, table, 1.0, 30.0), 1), 2 * vocab * h, hbm, "GB/s")
        # K2: a prefill product (2,048 rows, gate|up with SwiGLU).
        rows2k = draw(PREFILL_TOKENS, h)
        out["k2_prefill_product"] = record(timed(lambda i: ops.linear_swiglu(rows2k, weights[i]), 6),
                                           2.0 * PREFILL_TOKENS * 2 * inner * h, tensor, "TFLOP/s")
        del weights
        # K6 / K5: attention over a paged cache of random values, pages in order.
        def attention(batch: int, q_len: int, context: int):
            pages_per = -(-context // 16)
            sets = max(2, int(200e6 // (batch * pages_per * 2 * nkv * 16 * d * 2)) + 1)
            caches = [draw(batch * pages_per, 2, nkv, 16, d) for _ in range(sets)]
            i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=device)
            table = torch.arange(batch * pages_per, dtype=torch.int32, device=device).view(batch, pages_per)
            tokens = batch * q_len
            step = StepContext(
                num_tokens=tokens, num_seqs=batch, token_ids=i32([0] * tokens),
                positions=i32([context - q_len + t for _ in range(batch) for t in range(q_len)]),
                cu_seqlens=i32([q_len * b for b in range(batch + 1)]), seq_lens=i32([context] * batch),
                state_slots=i32([0] * batch), fresh=i32([0] * batch), logit_rows=i32([]), q_lens=[q_len] * batch,
                seq_lens_host=[context] * batch, max_q_len=q_len, max_seq_len=context, decode_only=q_len == 1,
                groups={}, workspace={"private": True})
            q, gate = draw(tokens, nq, d) * 20, draw(tokens, nq * d)
            slots = torch.zeros(tokens, dtype=torch.int64, device=device)
            seconds = timed(lambda i: ops.paged_attention(q, KVView(caches[i], table, slots, 16, None), step,
                                                          d ** -0.5, gate=gate), sets)
            return seconds

        out["k6_decode_attention"] = record(attention(args.batch, 1, args.context),
                                            args.batch * args.context * 2 * nkv * d * 2, hbm, "GB/s")
        out["k5_prefill_attention"] = record(attention(1, PREFILL_TOKENS, PREFILL_TOKENS),
                                             4.0 * nq * d * PREFILL_TOKENS * (PREFILL_TOKENS + 1) / 2, tensor, "TFLOP/s")
        return out

    if args.timeline:
        # One step of a tracing build, kernel by kernel as it runs (set OMNIA_TIMELINE=1): the lines
        # go to stderr, the record says how many kernels were seen.
        from mlx_omnia_b200.kernels import timeline
        if args.only == "prefill":
            prefill(args.prefill_tokens, 1, 2)
            torch.cuda.synchronize()
            timeline.spans()
            prefill(args.prefill_tokens, 1, 0)
            anchor = "attention_tcgen05"
        elif args.only == "mixed":
            # Eager steps (a captured shape would be replayed without passing the host-side marks).
            decoders = [engine.cache.open(f"mixed-{i}") for i in range(args.batch)]
            reader = engine.cache.open("mixed-reader")
            if decoders:
                engine.runner.run([StepEntry(r, p, []) for r, p in zip(decoders, prompts(args.batch, args.context - 4))])
            graphs, engine.runner.mixed_graphs = getattr(engine.runner, "mixed_graphs", None), None
            for index in range(3):
                if index == 2:
                    torch.cuda.synchronize()
                    timeline.spans()
                engine.runner.run([StepEntry(r, [1 + index], [0]) for r in decoders] +
                                  [StepEntry(reader, prompts(1, args.portion)[0], [])])
            engine.runner.mixed_graphs = graphs
            anchor = "attention_tcgen05"
        else:
            length = args.context - 16
            generator = Generator(engine, max_tokens_per_step=args.batch * length)
            for p in prompts(args.batch, length):
                generator.add(p, GenerationOptions(max_tokens=12, stop=()))
            for _ in range(6):
                generator.step()
            torch.cuda.synchronize()
            timeline.spans()
            generator.step()
            anchor = "attention_tc"
        torch.cuda.synchronize()
        kernels = timeline.spans()
        print("\n".join(timeline.by_layer(kernels, anchor)), file=sys.stderr)
        return {"only": args.only, "timeline": True, "kernels": len(kernels), "layers": layers}
    if args.only == "decode":  # a small case for profilers: one batch size, no prefill timing
        part = decode(args.batch, args.steps, args.warmup)
        step_bytes = weight_bytes + args.batch * part["context"] * kv_per_token
        return {"only": "decode", "config": args.config, "batch": args.batch, "layers": layers,
                "ms_per_step": round(part["ms"], 4), "tokens_per_s": round(part["tokens_per_s"], 1),
                "context": part["context"], "step_gb": round(step_bytes / 1e9, 2),
                "hbm_frac": round(step_bytes / (part["ms"] / 1e3) / 1e9 / measured["hbm_gbs"], 3)}
    def replayed(body, sets: int, rounds: int = 10) -> float:
        """Microseconds per call of `body(i)`, i over `sets` operand sets, replayed from a graph."""
        side = torch.cuda.Stream()
        with torch.cuda.stream(side):
            for i in range(sets):
                body(i)
            torch.cuda.synchronize()
            graph = torch.cuda.CUDAGraph()
            with capturing(graph, stream=side):
                for i in range(sets):
                    body(i)
        torch.cuda.synchronize()
        graph.replay()
        start, stop = events()
        start.record()
        for _ in range(rounds):
            graph.replay()
        stop.record()
        torch.cuda.synchronize()
        return start.elapsed_time(stop) * 1e3 / (rounds * sets)

    if args.only == "portions":
        # Prompts read in portions (a token budget): milliseconds for the whole prompt, with the attention
        # kernel's blocks cut into parts as the dispatch cuts them, and whole (no part shorter than a
        # million tiles).
        record = {"only": "portions", "config": args.config, "layers": layers, "unit": "ms"}
        kept = ops.PREFILL_MIN_PART_TILES
        for label, least in (("in_parts", kept), ("whole_blocks", 10 ** 6)):
            ops.PREFILL_MIN_PART_TILES = least
            record[label] = {f"{total}_in_{portion}": round(portions(total, portion), 2)
                             for total, portion in ((8192, 512), (8192, 256), (32768, 1024), (32768, 512))}
        ops.PREFILL_MIN_PART_TILES = kept
        ops.raise_on_error(engine.runtime.device)
        return record
    if args.only == "products":
        # A layer's four products at several row counts: this package's kernels (the streaming kernel up
        # to 16 rows, the one-SM and the two-SM tcgen05 kernels) beside the vendor library's product
        # (followed by the SwiGLU kernel for gate|up); weights fresh for every launch.
        device = engine.runtime.device
        h, inner = text["hidden_size"], text["intermediate_size"]
        q, kv = text["num_attention_heads"] * text["head_dim"], text["num_key_value_heads"] * text["head_dim"]
        shapes = {"qkv": (2 * q + 2 * kv, h, 0), "o": (h, q, 0), "gate_up": (2 * inner, h, 1), "down": (h, inner, 0)}
        draw = lambda *shape: torch.randn(*shape, device=device, dtype=torch.bfloat16) * 0.05
        table = {}
        for rows in (8, 16, 32, 64, 128, 264, 512, 1024, 2048, 4096, 8192):
            for name, (n, k, epilogue) in shapes.items():
                weights, a = [draw(n, k) for _ in range(6)], draw(rows, k) * 20
                out = torch.empty(rows, n // 2 if epilogue else n, dtype=torch.bfloat16, device=device)
                def library(i):
                    z = torch.mm(a, weights[i].t())
                    return ops.swiglu(z) if epilogue else z
                entry = {"library": round(replayed(library, 6), 1)}
                if rows <= 16:
                    entry["streaming"] = round(replayed(lambda i: ops._gemv_stream(a, weights[i], out, epilogue), 6), 1)
                if rows >= 128:
                    entry["one_sm"] = round(replayed(lambda i: ops._gemm_tcgen05(a, weights[i], out, epilogue, pair=False), 6), 1)
                if rows >= 256:
                    entry["two_sm"] = round(replayed(lambda i: ops._gemm_tcgen05(a, weights[i], out, epilogue, pair=True), 6), 1)
                table[f"{name}_{rows}"] = entry
        ops.raise_on_error(device)
        return {"only": "products", "config": args.config, "unit": "us", "products": table}
    if args.only == "elementwise":
        # The prefill step's element-wise kernels alone, buffers fresh for every launch.
        from mlx_omnia_b200.parts.base import KVView
        device = engine.runtime.device
        tokens, h, d = args.prefill_tokens, text["hidden_size"], text["head_dim"]
        nq, nkv = text["num_attention_heads"], text["num_key_value_heads"]
        xs = [torch.randn(tokens, h, device=device) for _ in range(8)]
        branches = [torch.randn(tokens, h, device=device).bfloat16() for _ in range(8)]
        wb, wo = torch.rand(h, device=device) + 0.5, torch.rand(h, device=device) + 0.5
        residual = replayed(lambda i: ops.add_rmsnorm(xs[i], branches[i], wb, 1e-6, wo, 1e-6), 8)
        rows = [torch.randn(tokens, (2 * nq + 2 * nkv) * d, device=device).bfloat16() for _ in range(8)]
        pages = [torch.zeros(-(-tokens // 16), 2, nkv, 16, d, device=device, dtype=torch.bfloat16) for _ in range(8)]
        inv_freq = 1.0 / (1e6 ** (torch.arange(0, d, 2, device=device).float() / d))
        positions = torch.arange(tokens, device=device, dtype=torch.int32)
        slots = torch.arange(tokens, device=device, dtype=torch.int64)
        blocks = torch.arange(-(-tokens // 16), device=device, dtype=torch.int32).view(1, -1)
        rope = replayed(lambda i: ops.qk_norm_rope_store(rows[i], 0, 2 * nq * d, (2 * nq + nkv) * d, nq, nkv, d, 1e-6, inv_freq,
                                                         positions, KVView(pages[i], blocks, slots, 16, None)), 8)
        moved = {"add_rmsnorm": tokens * h * (4 + 2 + 4 + 2), "qk_norm_rope_store": tokens * (nq + 2 * nkv) * d * 2 * 2}
        ops.raise_on_error(device)
        return {"only": "elementwise", "config": args.config, "tokens": tokens,
                "add_rmsnorm": {"us": round(residual, 2), "frac": round(moved["add_rmsnorm"] / residual / 1e3 / measured["hbm_gbs"], 3)},
                "qk_norm_rope_store": {"us": round(rope, 2),
                                       "frac": round(moved["qk_norm_rope_store"] / rope / 1e3 / measured["hbm_gbs"], 3)}}
    if args.only == "sampling":  # temperature, top-k and top-p over the full vocabulary, one row a request
        rows = args.batch
        logits = torch.randn(rows, vocab, device=engine.runtime.device, dtype=torch.float32) * 2.0
        f32 = lambda v: torch.full((rows,), v, dtype=torch.float32, device=logits.device)
        top_k = torch.full((rows,), 50, dtype=torch.int32, device=logits.device)
        seeds = torch.arange(rows, dtype=torch.int64, device=logits.device)
        call = lambda: ops.sample(logits, f32(0.8), top_k, f32(0.95), f32(0.0), seeds, seeds)
        for _ in range(max(args.warmup, 1)):
            call()
        start, stop = events()
        start.record()
        for _ in range(args.steps):
            call()
        stop.record()
        torch.cuda.synchronize()
        return {"only": "sampling", "rows": rows, "vocab": vocab, "us": round(start.elapsed_time(stop) * 1e3 / args.steps, 2)}
    if args.only == "mixed":
        part = mixed(args.batch, args.portion, args.steps, max(args.warmup, 4))
        return {"only": "mixed", "decoders": args.batch, "portion": args.portion, "layers": layers,
                "ms": round(part["ms"], 3), "host_ms": round(part["wall_ms"], 3)}
    if args.only == "prefill":
        part = prefill(args.prefill_tokens, args.steps, args.warmup)
        return {"only": "prefill", "config": args.config, "layers": layers, "tokens": args.prefill_tokens,
                "ms": round(part["ms"], 3), "frac": round(part["frac"], 4)}
    with ClockSampler() as sampler:
        main = decode(args.batch, args.steps, args.warmup)
    clocks = sampler.summary()
    side_steps = max(8, min(args.steps, 32))
    points = {f"decode_b{b}": round(decode(b, side_steps, 3)["tokens_per_s"], 1) for b in (1, 64)}
    pre = prefill(PREFILL_TOKENS, 5, 3)
    for name, (decoders, portion) in {"mixed_b8_ctx4096_portion256": (8, 256), "mixed_portion128": (0, 128)}.items():
        # (Four untimed steps: the prompt's first portion has a shape of its own, the shape of the others
        # is captured at its third coming.)
        part = mixed(decoders, portion, 8 if decoders else 4, 4)  # (a lone prompt of 8 x 128 tokens keeps its table width)
        points[name + "_ms"] = round(part["ms"], 3)
        points[name + "_host_ms"] = round(part["wall_ms"], 3)
    points["prefill_8192_in_portions_of_512_ms"] = round(portions(8192, 512), 2)
    kernels = kernel_classes()
    ops.raise_on_error(engine.runtime.device)

    step_bytes = weight_bytes + args.batch * main["context"] * kv_per_token
    achieved = step_bytes / (main["ms"] / 1000.0) / 1e9
    h2d = 4 * (3 * args.batch + (args.batch + 1) + 2 * args.batch) + 8 * args.batch + \
        4 * args.batch * -(-main["context"] // 16)
    # What a replayed decode step really copies: the whole metadata buffer of its graph, whose block
    # tables are as wide as the graph's bucket, not as the requests' own.
    graphs = getattr(engine.runner, "graphs", None)
    bucket = 1 << max(args.batch - 1, 0).bit_length()
    copied = [c.host_tensor.numel() * 4 for c in graphs.captured.values() if c.layout.seqs == bucket] \
        if graphs is not None else []
    if copied:
        h2d = int(max(copied))
    return {
        "metric": "decode tok/s at batch 8 (configs[2], context 4096)", "value": round(main["tokens_per_s"], 1),
        "unit": "tokens/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": round(main["ms"], 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic: seeded uniform-random token ids, random weights N(0, 0.02)",
        "config": {"model": "muse_glimmer configs[2]", "layers": layers, "layers_full": full_layers,
                   "hidden": text["hidden_size"], "heads": text["num_attention_heads"],
                   "kv_heads": text["num_key_value_heads"], "head_dim": text["head_dim"],
                   "intermediate": text["intermediate_size"], "vocab": vocab, "tied": True, "global_batch": args.batch,
                   "seq_len": args.context, "context_at_timed_steps": main["context"], "page_size": 16,
                   "params": params, "parallelism": "single-gpu", "l2": f"weights ({weight_bytes / 1e9:.1f} GB) exceed L2; no flush",
                   "peaks": peak_source},
        "clocks": clocks,
        "e2e": {"value": round(main["wall_tokens_per_s"], 1), "unit": "tokens/s", "h2d_bytes_per_step": h2d,
                "d2h_bytes_per_step": 4 * args.batch},
        "gpu_launches": main["launches"] * args.steps,
        "prefill": {"value": round(pre["value"], 1), "tokens": pre["tokens"], "ms": round(pre["ms"], 3),
                    "frac": round(pre["frac"], 4)},
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": measured["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / measured["hbm_gbs"], 4)},
        "points": points,
        "kernels": kernels,
    }


FOKALORN_SIZES = {
    # width, feed-forward, heads (of 128), layers, latent rank, rotated dims, streams, norm groups
    "1024": dict(width=1024, ff=3072, heads=8, layers=8, rank=256, rot=64, streams=2, groups=4),
    "2048": dict(width=2048, ff=6144, heads=16, layers=8, rank=512, rot=64, streams=4, groups=8),
    "4096": dict(width=4096, ff=12288, heads=32, layers=4, rank=512, rot=64, streams=4, groups=8),
}
FOKALORN_VOCAB = 32768


def fokalorn_config(size: dict) -> dict:
    """Three recurrent layers to one of latent attention, every layer with a feed-forward."""
    delta = {"type": "channel_delta", "mlp": {"ff": size["ff"], "kind": "dense"},
             "mixer": {"heads": size["heads"], "kv_heads": size["heads"], "dim": 128, "vdim": 128, "conv": 4,
                       "decay_rank": 64, "gate_rank": 64}}
    latent = {"type": "latent_attention", "mlp": {"ff": size["ff"], "kind": "dense"},
              "mixer": {"heads": size["heads"], "dim": 128, "rot_dim": size["rot"], "vdim": 128, "kv_rank": size["rank"],
                        "scale": (128 + size["rot"]) ** -0.5, "rot": {"base": 10000.0, "dims": size["rot"]}}}
    layers = [json.loads(json.dumps(latent if i % 4 == 3 else delta)) for i in range(size["layers"])]
    return {"architecture": "Fokalorn", "vocab": FOKALORN_VOCAB, "width": size["width"], "embedding": {"scale": 1.0},
            "norm": {"eps": 1e-5, "groups": size["groups"]}, "streams": size["streams"], "layers": layers}


def muse_config_like(size: dict) -> dict:
    raw = json.loads(json.dumps(CONFIG2))
    n = size["layers"]
    raw["text_config"].update(hidden_size=size["width"], intermediate_size=size["ff"], num_hidden_layers=n,
                              num_attention_heads=size["heads"], num_key_value_heads=max(size["heads"] // 2, 1),
                              vocab_size=FOKALORN_VOCAB, layer_types=["full_attention"] * n,
                              layer_rope_theta=[1000000.0] * n, tie_word_embeddings=False)
    return raw


def run_fokalorn(args) -> dict:
    """Prefill (one prompt of --prefill-tokens) and decode (--batch requests ending at --context tokens)
    of Fokalorn and of Muse-Glimmer at equal sizes, then the new design's kernels alone."""
    import torch

    from mlx_omnia_b200.engine.engine import Engine, EngineArgs
    from mlx_omnia_b200.engine.step import StepEntry
    from mlx_omnia_b200.kernels import ops

    measured, peak_source = peaks()
    hbm, flops_peak = measured["hbm_gbs"] * 1e9, measured["bf16_tflops"] * 1e12
    g = torch.Generator().manual_seed(SEED)
    steps, warmup, batch, context, tokens = args.steps, max(args.warmup, 3), args.batch, args.context, args.prefill_tokens

    def timed(fn, count, warm=3):
        for _ in range(warm):
            fn()
        torch.cuda.synchronize()
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        for _ in range(count):
            fn()
        stop.record()
        torch.cuda.synchronize()
        return start.elapsed_time(stop) / count

    def whole_model(raw) -> dict:
        engine = Engine.from_random(raw, SEED, EngineArgs(dtype="bfloat16", page_size=16, max_requests=batch + 1,
                                                          cache_tokens=batch * (context + 16) + tokens + 16))
        times = []
        for index in range(warmup + 3):
            request = engine.cache.open(f"p{index}")
            ids = torch.randint(0, FOKALORN_VOCAB, (tokens,), generator=g).tolist()
            torch.cuda.synchronize()
            start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record()
            engine.runner.run([StepEntry(request, ids, [tokens - 1])])
            stop.record()
            torch.cuda.synchronize()
            engine.cache.close(request.request_id)
            times.append(start.elapsed_time(stop))
        prefill_ms = statistics.median(times[warmup:])
        requests = [engine.cache.open(f"d{i}") for i in range(batch)]
        length = context - steps - warmup - 1
        for r in requests:  # one prompt a step: a step of every prompt would need scratch for batch x length rows
            engine.runner.run([StepEntry(r, torch.randint(0, FOKALORN_VOCAB, (length,), generator=g).tolist(), [])])
        entries = lambda i: [StepEntry(r, [1 + i], [0]) for r in requests]
        for i in range(warmup):
            engine.runner.run(entries(i), copy=False)
        torch.cuda.synchronize()
        launches = ops.launches
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        for i in range(steps):
            engine.runner.run(entries(warmup + i), copy=False)
        stop.record()
        torch.cuda.synchronize()
        decode_ms = start.elapsed_time(stop) / steps
        ops.raise_on_error(engine.runtime.device)
        weights = sum(t.numel() * t.element_size() for t in _model_tensors(engine.model))
        out = {"prefill_tokens_per_s": round(tokens * 1000.0 / prefill_ms, 1), "prefill_ms": round(prefill_ms, 3),
               "decode_tokens_per_s": round(batch * 1000.0 / decode_ms, 1), "decode_ms": round(decode_ms, 4),
               "launches_per_decode_step": (ops.launches - launches) // steps, "weight_gb": round(weights / 1e9, 3)}
        for r in requests:
            engine.cache.close(r.request_id)
        del engine
        torch.cuda.empty_cache()
        return out

    def _model_tensors(model):
        seen, out, stack = set(), [], [model]
        while stack:
            item = stack.pop()
            if isinstance(item, torch.Tensor):
                if item.is_cuda and item.data_ptr() not in seen:
                    seen.add(item.data_ptr())
                    out.append(item)
            elif isinstance(item, (list, tuple)):
                stack.extend(item)
            elif isinstance(item, dict):
                stack.extend(item.values())
            elif hasattr(item, "__dict__") and type(item).__module__.startswith("mlx_omnia_b200.parts"):
                stack.extend(v for k, v in vars(item).items() if k != "runtime")
        return out

    def kernels(size: dict) -> dict:
        """Each kernel of the new design alone, at this size, with the bytes or FLOPs it cannot avoid;
        and Muse-Glimmer's like kernels at the same heads. Times are per launch over `reps` launches
        on operands larger than L2 where the operands are large at all."""
        from mlx_omnia_b200.parts.base import KVSpec, KVView

        dev, bf = torch.device("cuda:0"), torch.bfloat16
        H, D, rank, rot, S = size["heads"], size["width"], size["rank"], size["rot"], size["streams"]
        dk = dv = 128
        out = {}

        class Step:
            pass

        def step_of(lens, starts):
            st = Step()
            st.num_seqs, st.q_lens = len(lens), list(lens)
            cu = [0]
            for n in lens:
                cu.append(cu[-1] + n)
            st.cu_seqlens = torch.tensor(cu, dtype=torch.int32, device=dev)
            st.state_slots = torch.arange(len(lens), dtype=torch.int32, device=dev)
            st.positions = torch.tensor([s + i for s, n in zip(starts, lens) for i in range(n)], dtype=torch.int32, device=dev)
            st.seq_lens = torch.tensor([s + n for s, n in zip(starts, lens)], dtype=torch.int32, device=dev)
            st.seq_lens_host, st.max_q_len, st.max_seq_len = [s + n for s, n in zip(starts, lens)], max(lens), max(s + n for s, n in zip(starts, lens))
            st.decode_only, st.workspace = all(n == 1 for n in lens), None
            return st

        def note(name, ms, bytes_=None, flops=None, like=None):
            entry = {"us": round(ms * 1000.0, 2)}
            if bytes_ is not None:
                entry.update(gb_s=round(bytes_ / ms / 1e6, 1), frac_hbm=round(bytes_ / (ms / 1e3) / hbm, 4))
            if flops is not None:
                entry.update(tflops=round(flops / ms / 1e9, 2), frac_tensor=round(flops / (ms / 1e3) / flops_peak, 4))
            out[name] = entry

        for mode, lens, starts in (("prefill", [tokens], [0]), ("decode", [1] * batch, [context - 1] * batch)):
            st = step_of(lens, starts)
            T = sum(lens)
            # the recurrent mixer's kernels
            C = 2 * H * dk + H * dv
            proj = torch.randn(T, C + H, device=dev).to(bf)
            taps = torch.randn(C, 4, device=dev)
            conv_state = torch.zeros(len(lens) + 1, 3, C, device=dev)
            S_state = torch.zeros(len(lens) + 1, H, dk, dv, device=dev)
            a, gate = torch.randn(T, H * dk, device=dev).to(bf), torch.randn(T, H * dv, device=dev).to(bf)
            A_log, dt_bias, nw = torch.zeros(H, device=dev), torch.zeros(H * dk, device=dev), torch.ones(dv, device=dev)
            run_conv = lambda: ops.short_conv(proj, 0, C, taps, conv_state, st, 2 * H * dk, dk, 1e-6, H * dk, dk ** -0.5,
                                              a, A_log, dt_bias, C, H)
            conv = run_conv()
            note(f"short_conv_{mode}", timed(run_conv, 20), bytes_=T * (C * (2 + 4) + H * dk * (2 + 4)))
            ms = timed(lambda: ops.delta_rule(conv, C, H, H, dk, dv, proj, 0, gate, nw, 1e-5, S_state, conv_state, 4, st), 20)
            state_bytes = 2 * len(lens) * H * dk * dv * 4
            note(f"delta_rule_{mode}", ms, bytes_=state_bytes + T * ((C + H * dk) * 4 + 2 * H * dv * 2),
                 flops=T * H * dk * dv * 2 * 3)
            # latent attention's kernels
            page, width = 16, rank + rot
            pages = -(-st.max_seq_len // page)
            cache = (torch.randn(len(lens) * pages, 1, 1, page, width, device=dev) * 0.3).to(bf)
            table = torch.arange(len(lens) * pages, dtype=torch.int32, device=dev).view(len(lens), pages)
            slots = torch.cat([table[i].long()[(st.positions[st.cu_seqlens[i]: st.cu_seqlens[i + 1]] // page).long()] * page
                               + st.positions[st.cu_seqlens[i]: st.cu_seqlens[i + 1]].long() % page for i in range(len(lens))])
            kv = KVView(cache, table, slots, page, None, True, KVSpec(((1, width),)))
            qd = 128 + rot
            lproj = (torch.randn(T, H * qd + width + H, device=dev) * 0.3).to(bf)
            inv = torch.tensor([10000.0 ** (-2.0 * i / rot) for i in range(rot // 2)], device=dev)
            dn_w = torch.ones(rank, device=dev)
            ms = timed(lambda: ops.latent_prepare(lproj, 0, H, qd, H * qd, rank, rot, dn_w, 1e-5, inv, st.positions, kv), 20)
            note(f"latent_prepare_{mode}", ms, bytes_=T * (2 * width + 2 * H * rot) * 2)
            q_lat = (torch.randn(H, T, rank, device=dev) * 0.1).to(bf)
            o_lat = torch.empty(H, T, rank, dtype=bf, device=dev)
            q_rot = lproj[:, : H * qd].view(T, H, qd)[:, :, 128:]
            sink = torch.zeros(H, device=dev)
            reps = 3 if mode == "prefill" else 10
            ms = timed(lambda: ops.latent_attention(q_lat, q_rot, kv, st, 0.07, sink, lproj[:, H * qd + width:], o_lat), reps, 1)
            pairs = sum(s * n + n * (n + 1) // 2 for s, n in zip(starts, lens))
            note(f"latent_attention_{mode}", ms, bytes_=sum(s + n for s, n in zip(starts, lens)) * width * 2 + 4 * T * H * rank,
                 flops=2 * pairs * H * (width + rank))
            # the residual streams' kernels, and the residual step of a single stream beside them
            xs = torch.randn(T, S * D, device=dev)
            y = torch.randn(T, D, device=dev).to(bf)
            coef, mix, outc, w = torch.ones(S, device=dev), torch.eye(S, device=dev), torch.ones(S, device=dev), torch.ones(D, device=dev)
            ms = timed(lambda: ops.streams_enter(xs, coef, S, w, 1e-5, size["groups"], bf), 20)
            note(f"streams_enter_{mode}", ms, bytes_=T * (S * D * 4 + D * 2))
            ms = timed(lambda: ops.streams_leave(xs, y, mix, outc, S), 20)
            note(f"streams_leave_{mode}", ms, bytes_=T * (2 * S * D * 4 + D * 2))
            x1 = torch.randn(T, D, device=dev)
            ms = timed(lambda: ops.add_rmsnorm(x1, y, None, None, w, 1e-5), 20)
            note(f"like:add_rmsnorm_{mode}", ms, bytes_=T * (2 * D * 4 + 2 * D * 2))
            # Muse-Glimmer's attention at the same heads (half as many key/value heads, head size 128)
            nkv = max(H // 2, 1)
            gcache = (torch.randn(len(lens) * pages, 2, nkv, page, 128, device=dev) * 0.3).to(bf)
            gkv = KVView(gcache, table, slots, page, None, True, KVSpec.keys_and_values(nkv, 128))
            q = (torch.randn(T, H, 128, device=dev) * 0.3).to(bf)
            ms = timed(lambda: ops.paged_attention(q, gkv, st, 0.09), 10, 2)
            note(f"like:paged_attention_{mode}", ms, bytes_=sum(s + n for s, n in zip(starts, lens)) * 2 * nkv * 128 * 2 + 4 * T * H * 128,
                 flops=2 * pairs * H * 256)
        ops.raise_on_error(dev)
        return out

    record = {"metric": "Fokalorn beside Muse-Glimmer at equal sizes", "unit": "tokens/s", "dtype": "bf16",
              "data": "synthetic: seeded uniform-random token ids, random weights",
              "config": {"prefill_tokens": tokens, "decode_batch": batch, "decode_context": context, "vocab": FOKALORN_VOCAB,
                         "peaks": peak_source}, "sizes": {}}
    for name in ([args.size] if args.size else list(FOKALORN_SIZES)):
        size = FOKALORN_SIZES[name]
        record["sizes"][name] = {"fokalorn": whole_model(fokalorn_config(size)),
                                 "muse_glimmer": whole_model(muse_config_like(size)),
                                 "kernels": kernels(size), "layers": size["layers"]}
    return record


DOLUTAR_SIZES = {
    # width, heads x head size, key/value heads, layers, window and kept positions, the dense layer's
    # feed-forward, experts (with tensors + identity) of which `top` a token, an expert's feed-forward
    "1024": dict(width=1024, heads=16, dim=64, kv=4, layers=8, window=512, keep=64, ff=4096, experts=16, identity=2, top=2, eff=1024),
    "2048": dict(width=2048, heads=16, dim=128, kv=4, layers=8, window=512, keep=64, ff=8192, experts=32, identity=4, top=4, eff=1536),
    "4096": dict(width=4096, heads=32, dim=128, kv=8, layers=4, window=1024, keep=128, ff=12288, experts=16, identity=2, top=4, eff=2048),
}
DOLUTAR_VOCAB = 32768


def dolutar_config(size: dict) -> dict:
    """The first layer with the dense feed-forward, the others routed; every second layer reads the
    cache of the layer before it."""
    layers = []
    for i in range(size["layers"]):
        mixer = {"heads": size["heads"], "kv_heads": size["kv"], "dim": size["dim"], "vdim": size["dim"],
                 "scale": size["dim"] ** -0.5, "rot": {"base": 100000.0, "dims": size["dim"]},
                 "mask": {"size": size["window"], "keep_first": size["keep"]}}
        if i % 2 == 1:
            mixer["kv_from"] = i - 1
        mlp = {"kind": "dense", "ff": size["ff"], "limit": 7.0} if i == 0 else \
            {"kind": "moe", "expert": {"ff": size["eff"]},
             "router": {"experts": size["experts"], "identity": size["identity"], "top": size["top"]}}
        layers.append({"type": "attention", "mixer": mixer, "mlp": mlp})
    return {"architecture": "Dolutar", "vocab": DOLUTAR_VOCAB, "width": size["width"], "logit_scale": 1.0,
            "norm": {"eps": 1e-5}, "embedding": {"scale": 1.0, "bigram": {"buckets": 65521, "mul_prev": 131, "mul_cur": 17}},
            "layers": layers}


def muse_config_like_dolutar(size: dict) -> dict:
    """Muse-Glimmer with sliding attention at the same width, depth, heads and window; its feed-forward
    as wide as the experts one token of the routed design uses."""
    raw = json.loads(json.dumps(CONFIG2))
    n = size["layers"]
    raw["text_config"].update(hidden_size=size["width"], intermediate_size=size["top"] * size["eff"], num_hidden_layers=n,
                              num_attention_heads=size["heads"], num_key_value_heads=size["kv"], head_dim=size["dim"],
                              vocab_size=DOLUTAR_VOCAB, layer_types=["sliding_attention"] * n, sliding_window=size["window"],
                              layer_rope_theta=[100000.0] * n, tie_word_embeddings=False)
    return raw


def run_dolutar(args) -> dict:
    """Prefill (one prompt of --prefill-tokens) and decode (--batch requests ending at --context tokens)
    of Dolutar and of Muse-Glimmer at equal sizes, then the new design's kernels alone, each beside the
    like kernel of Muse-Glimmer."""
    import torch

    from mlx_omnia_b200.engine.engine import Engine, EngineArgs
    from mlx_omnia_b200.engine.step import StepEntry
    from mlx_omnia_b200.kernels import ops
    from mlx_omnia_b200.parts.base import KVSpec, KVView

    measured, peak_source = peaks()
    hbm, flops_peak = measured["hbm_gbs"] * 1e9, measured["bf16_tflops"] * 1e12
    g = torch.Generator().manual_seed(SEED)
    steps, warmup, batch, context, tokens = args.steps, max(args.warmup, 3), args.batch, args.context, args.prefill_tokens
    dev, bf = torch.device("cuda:0"), torch.bfloat16

    def timed(fn, count, warm=3):
        for _ in range(warm):
            fn()
        torch.cuda.synchronize()
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        for _ in range(count):
            fn()
        stop.record()
        torch.cuda.synchronize()
        return start.elapsed_time(stop) / count

    def whole_model(raw) -> dict:
        engine = Engine.from_random(raw, SEED, EngineArgs(dtype="bfloat16", page_size=16, max_requests=batch + 1,
                                                          cache_tokens=batch * (context + 16) + tokens + 16))
        times = []
        for index in range(warmup + 3):
            request = engine.cache.open(f"p{index}")
            ids = torch.randint(0, DOLUTAR_VOCAB, (tokens,), generator=g).tolist()
            torch.cuda.synchronize()
            start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record()
            engine.runner.run([StepEntry(request, ids, [tokens - 1])])
            stop.record()
            torch.cuda.synchronize()
            engine.cache.close(request.request_id)
            times.append(start.elapsed_time(stop))
        prefill_ms = statistics.median(times[warmup:])
        requests = [engine.cache.open(f"d{i}") for i in range(batch)]
        length = context - steps - warmup - 1
        for r in requests:
            engine.runner.run([StepEntry(r, torch.randint(0, DOLUTAR_VOCAB, (length,), generator=g).tolist(), [])])
        entries = lambda i: [StepEntry(r, [1 + i], [0]) for r in requests]
        for i in range(warmup):
            engine.runner.run(entries(i), copy=False)
        torch.cuda.synchronize()
        launches = ops.launches
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        for i in range(steps):
            engine.runner.run(entries(warmup + i), copy=False)
        stop.record()
        torch.cuda.synchronize()
        decode_ms = start.elapsed_time(stop) / steps
        ops.raise_on_error(engine.runtime.device)
        out = {"prefill_tokens_per_s": round(tokens * 1000.0 / prefill_ms, 1), "prefill_ms": round(prefill_ms, 3),
               "decode_tokens_per_s": round(batch * 1000.0 / decode_ms, 1), "decode_ms": round(decode_ms, 4),
               "launches_per_decode_step": (ops.launches - launches) // steps}
        for r in requests:
            engine.cache.close(r.request_id)
        del engine
        torch.cuda.empty_cache()
        return out

    class Step:
        pass

    def step_of(lens, starts):
        st = Step()
        st.num_seqs, st.q_lens = len(lens), list(lens)
        cu = [0]
        for n in lens:
            cu.append(cu[-1] + n)
        st.num_tokens = cu[-1]
        st.cu_seqlens = torch.tensor(cu, dtype=torch.int32, device=dev)
        st.state_slots = torch.arange(len(lens), dtype=torch.int32, device=dev)
        st.positions = torch.tensor([s + i for s, n in zip(starts, lens) for i in range(n)], dtype=torch.int32, device=dev)
        st.seq_lens = torch.tensor([s + n for s, n in zip(starts, lens)], dtype=torch.int32, device=dev)
        st.seq_lens_host, st.max_q_len = [s + n for s, n in zip(starts, lens)], max(lens)
        st.max_seq_len = max(st.seq_lens_host)
        st.decode_only, st.workspace = all(n == 1 for n in lens), None
        return st

    def kernels(size: dict) -> dict:
        H, G, d, D = size["heads"], size["kv"], size["dim"], size["width"]
        window, keep = size["window"], size["keep"]
        E, R, top, F = size["experts"], size["experts"] + size["identity"], size["top"], size["eff"]
        out = {}

        def note(name, ms, bytes_=None, flops=None):
            entry = {"us": round(ms * 1000.0, 2)}
            if bytes_ is not None:
                entry.update(gb_s=round(bytes_ / ms / 1e6, 1), frac_hbm=round(bytes_ / (ms / 1e3) / hbm, 4))
            if flops is not None:
                entry.update(tflops=round(flops / ms / 1e9, 2), frac_tensor=round(flops / (ms / 1e3) / flops_peak, 4))
            out[name] = entry

        for mode, lens, starts in (("prefill", [tokens], [0]), ("decode", [1] * batch, [context - 1] * batch)):
            st = step_of(lens, starts)
            T = sum(lens)
            page = 16
            pages = -(-st.max_seq_len // page)
            table = torch.arange(len(lens) * pages, dtype=torch.int32, device=dev).view(len(lens), pages)
            slots = torch.cat([table[i].long()[(st.positions[st.cu_seqlens[i]: st.cu_seqlens[i + 1]] // page).long()] * page
                               + st.positions[st.cu_seqlens[i]: st.cu_seqlens[i + 1]].long() % page for i in range(len(lens))])
            cache = (torch.randn(len(lens) * pages, 2, G, page, d, device=dev) * 0.3).to(bf)
            kv = KVView(cache, table, slots, page, window, True, KVSpec(((G, d), (G, d)), window, keep_first=keep))
            like_kv = KVView(cache, table, slots, page, window, True, KVSpec.keys_and_values(G, d, window))
            # the embedding with its pair table, beside the plain lookup
            st.token_ids = torch.randint(0, DOLUTAR_VOCAB, (T,), device=dev, dtype=torch.int32)
            emb, pairs = (torch.randn(n, D, device=dev).to(bf) for n in (DOLUTAR_VOCAB, 65522))
            prev = torch.zeros(len(lens) + 1, dtype=torch.int32, device=dev)
            note(f"embed_pair_{mode}", timed(lambda: ops.embed_pair(st, emb, pairs, prev, 1.0, 131, 17), 20), bytes_=T * D * (2 + 2 + 4))
            note(f"like:embed_rmsnorm_{mode}", timed(lambda: ops.embed_rmsnorm(st.token_ids, emb, 1e-6), 20), bytes_=T * D * (2 + 4))
            # bias, head norms, rotation and the cache write, beside the weightless form
            cols = (H + 2 * G) * d
            proj, bias = (torch.randn(T, cols, device=dev) * 0.5).to(bf), torch.randn(cols, device=dev).to(bf)
            wq = torch.ones(d, device=dev)
            inv = torch.tensor([100000.0 ** (-2.0 * i / d) for i in range(d // 2)], device=dev)
            ms = timed(lambda: ops.qkv_prepare(proj, 0, H * d, (H + G) * d, H, d, bias, wq, wq, 1e-5, inv, st.positions, kv, True), 20)
            note(f"qkv_prepare_{mode}", ms, bytes_=T * cols * 4)
            ms = timed(lambda: ops.qk_norm_rope_store(proj, 0, H * d, (H + G) * d, H, G, d, 1e-5, inv, st.positions, like_kv), 20)
            note(f"like:qk_norm_rope_store_{mode}", ms, bytes_=T * cols * 4)
            # attention: window, kept positions and sink, beside the same window without them
            q = (torch.randn(T, H, d, device=dev) * 0.3).to(bf)
            sink = torch.zeros(H, device=dev)
            seen = sum(min(s + i + 1, window) for s, n in zip(starts, lens) for i in range(n))  # (query, key) pairs in the windows
            held = sum(min(s + n, window + n - 1) for s, n in zip(starts, lens))  # keys that are read at all
            reps = 5 if mode == "prefill" else 20
            ms = timed(lambda: ops.paged_attention(q, kv, st, d ** -0.5, sink=sink, window=window, keep_first=keep), reps, 2)
            note(f"sink_window_attention_{mode}", ms, bytes_=held * 2 * G * d * 2 + 4 * T * H * d, flops=4 * seen * H * d)
            ms = timed(lambda: ops.paged_attention(q, like_kv, st, d ** -0.5), reps, 2)
            note(f"like:paged_attention_{mode}", ms, bytes_=held * 2 * G * d * 2 + 4 * T * H * d, flops=4 * seen * H * d)
            # the residual step that also rounds the residual for the next reader, beside the one that norms it
            x1, y = torch.randn(T, D, device=dev), torch.randn(T, D, device=dev).to(bf)
            w = torch.ones(D, device=dev)
            note(f"add_norm_rounded_{mode}", timed(lambda: ops.add_rmsnorm(x1, y, w, 1e-5, None, None, rounded=True), 20),
                 bytes_=T * (2 * D * 4 + 2 * D * 2))
            note(f"like:add_rmsnorm_{mode}", timed(lambda: ops.add_rmsnorm(x1, y, w, 1e-5, w, 1e-5), 20), bytes_=T * (2 * D * 4 + 2 * D * 2))
            # the dense layer's clamped unit in its product, beside SwiGLU in the same product
            h = (torch.randn(T, D, device=dev) * 0.5).to(bf)
            gate_up = (torch.randn(2 * size["ff"], D, device=dev) * D ** -0.5).to(bf)
            dense = dict(bytes_=2 * size["ff"] * D * 2 + T * (D + size["ff"]) * 2, flops=2 * T * 2 * size["ff"] * D)
            note(f"linear_clamped_glu_{mode}", timed(lambda: ops.linear_clamped_glu(h, gate_up, 1.702, 7.0), 10), **dense)
            note(f"like:linear_swiglu_{mode}", timed(lambda: ops.linear_swiglu(h, gate_up), 10), **dense)
            del gate_up
            # routed experts: router, sorted order, the two grouped products, the weighted sum; beside the dense
            # feed-forward of the same active width (gate|up with SwiGLU, then down)
            router, correction = torch.randn(R, D, device=dev) * 0.05, torch.zeros(R, device=dev)
            egu = (torch.randn(E, 2 * F, D, device=dev) * D ** -0.5).to(bf)
            edn = (torch.randn(E, D, F, device=dev) * F ** -0.5).to(bf)
            counts = torch.zeros(E, dtype=torch.int32, device=dev)

            def route():
                counts.zero_()
                return ops.moe_route(h, router, correction, E, top, counts)

            note(f"moe_route_{mode}", timed(route, 20), bytes_=T * D * 2 + R * D * 4)
            ms = timed(lambda: ops.moe_experts(h, router, correction, egu, edn, top, st), 10)
            used = E * (1.0 - (1.0 - top / R) ** T)  # experts that T tokens' choices touch, on average
            note(f"moe_experts_{mode}", ms, bytes_=used * 3 * F * D * 2 + T * D * 4, flops=2 * T * top * 3 * F * D)
            dgu = (torch.randn(2 * top * F, D, device=dev) * D ** -0.5).to(bf)
            ddn = (torch.randn(D, top * F, device=dev) * (top * F) ** -0.5).to(bf)
            ms = timed(lambda: ops.linear(ops.linear_swiglu(h, dgu), ddn), 10)
            note(f"like:gated_mlp_{mode}", ms, bytes_=3 * top * F * D * 2 + T * D * 4, flops=2 * T * top * 3 * F * D)
            del egu, edn, dgu, ddn
        ops.raise_on_error(dev)
        return out

    record = {"metric": "Dolutar beside Muse-Glimmer (sliding attention) at equal sizes", "unit": "tokens/s", "dtype": "bf16",
              "data": "synthetic: seeded uniform-random token ids, random weights",
              "config": {"prefill_tokens": tokens, "decode_batch": batch, "decode_context": context, "vocab": DOLUTAR_VOCAB,
                         "peaks": peak_source}, "sizes": {}}
    for name in ([args.size] if args.size else list(DOLUTAR_SIZES)):
        size = DOLUTAR_SIZES[name]
        record["sizes"][name] = {"dolutar": whole_model(dolutar_config(size)),
                                 "muse_glimmer": whole_model(muse_config_like_dolutar(size)),
                                 "kernels": kernels(size), "layers": size["layers"]}
    return record


BOBARAX_SIZES = {
    # width, heads x head size (keys and values alike), key/value heads, layers, window of the windowed layers,
    # run length and cap of the run-masked layers, the dense feed-forward, experts of which `top` a token, an
    # expert's feed-forward; `keep` and `identity` only shape the Dolutar model beside it
    "1024": dict(width=1024, heads=16, dim=64, kv=4, layers=8, window=512, run=512, softcap=30.0, ff=4096, experts=16, top=2,
                 eff=1024, keep=64, identity=2),
    "2048": dict(width=2048, heads=16, dim=128, kv=4, layers=8, window=512, run=512, softcap=30.0, ff=8192, experts=32, top=4,
                 eff=1536, keep=64, identity=4),
    "4096": dict(width=4096, heads=32, dim=128, kv=8, layers=4, window=1024, run=1024, softcap=30.0, ff=12288, experts=16,
                 top=4, eff=2048, keep=128, identity=2),
}


def bobarax_config(size: dict) -> dict:
    """Layers in fours: a windowed layer with the dense feed-forward that owns a cache, a decayed
    linear-attention layer with experts, a run-masked layer with experts, and a windowed layer with
    experts that reads the first one's cache."""
    H, G, d = size["heads"], size["kv"], size["dim"]
    moe = {"kind": "moe", "expert": {"ff": size["eff"], "limit": 7.0}, "router": {"experts": size["experts"], "top": size["top"]}}
    windowed = {"heads": H, "kv_heads": G, "dim": d, "vdim": d, "scale": d ** -0.5, "rot": {"base": 100000.0, "dims": d // 2},
                "mask": {"size": size["window"]}}
    layers = []
    for i in range(size["layers"]):
        kind = i % 4
        if kind == 0:
            layers.append({"type": "attention_2", "mixer": dict(windowed), "mlp": {"kind": "dense", "ff": size["ff"]}})
        elif kind == 1:
            decay = [1.0 - 2.0 ** -(3 + 7 * h / max(H - 1, 1)) for h in range(H)]
            layers.append({"type": "lightning", "mixer": {"heads": H, "dim": d, "vdim": d, "decay": decay}, "mlp": moe})
        elif kind == 2:
            layers.append({"type": "attention", "mixer": {"heads": H, "kv_heads": G, "dim": d, "vdim": d, "scale": d ** -0.5,
                                                          "softcap": size["softcap"], "mask": {"size": size["run"]}}, "mlp": moe})
        else:
            layers.append({"type": "attention_2", "mixer": dict(windowed, kv_from=i - 3), "mlp": moe})
    return {"architecture": "Bobarax", "vocab": DOLUTAR_VOCAB, "width": size["width"], "residual_mult": 0.5, "logit_scale": 1.0,
            "norm": {"eps": 1e-5}, "layers": layers}


def run_bobarax(args) -> dict:
    """Prefill (one prompt of --prefill-tokens) and decode (--batch requests ending at --context tokens)
    of Bobarax and of Dolutar at equal sizes, then the new design's kernels alone, each beside the like
    kernel of Dolutar (attention, experts) or Fokalorn (the recurrence)."""
    import torch

    from mlx_omnia_b200.engine.engine import Engine, EngineArgs
    from mlx_omnia_b200.engine.step import StepEntry
    from mlx_omnia_b200.kernels import ops
    from mlx_omnia_b200.parts.base import KVSpec, KVView

    measured, peak_source = peaks()
    hbm, flops_peak = measured["hbm_gbs"] * 1e9, measured["bf16_tflops"] * 1e12
    g = torch.Generator().manual_seed(SEED)
    steps, warmup, batch, context, tokens = args.steps, max(args.warmup, 3), args.batch, args.context, args.prefill_tokens
    dev, bf = torch.device("cuda:0"), torch.bfloat16
    vocab = DOLUTAR_VOCAB

    def timed(fn, count, warm=3):
        for _ in range(warm):
            fn()
        torch.cuda.synchronize()
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        for _ in range(count):
            fn()
        stop.record()
        torch.cuda.synchronize()
        return start.elapsed_time(stop) / count

    def whole_model(raw) -> dict:
        engine = Engine.from_random(raw, SEED, EngineArgs(dtype="bfloat16", page_size=16, max_requests=batch + 1,
                                                          cache_tokens=batch * (context + 16) + tokens + 16))
        times = []
        for index in range(warmup + 3):
            request = engine.cache.open(f"p{index}")
            ids = torch.randint(0, vocab, (tokens,), generator=g).tolist()
            torch.cuda.synchronize()
            start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record()
            engine.runner.run([StepEntry(request, ids, [tokens - 1])])
            stop.record()
            torch.cuda.synchronize()
            engine.cache.close(request.request_id)
            times.append(start.elapsed_time(stop))
        prefill_ms = statistics.median(times[warmup:])
        requests = [engine.cache.open(f"d{i}") for i in range(batch)]
        length = context - steps - warmup - 1
        for r in requests:
            engine.runner.run([StepEntry(r, torch.randint(0, vocab, (length,), generator=g).tolist(), [])])
        entries = lambda i: [StepEntry(r, [1 + i], [0]) for r in requests]
        for i in range(warmup):
            engine.runner.run(entries(i), copy=False)
        torch.cuda.synchronize()
        launches = ops.launches
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        for i in range(steps):
            engine.runner.run(entries(warmup + i), copy=False)
        stop.record()
        torch.cuda.synchronize()
        decode_ms = start.elapsed_time(stop) / steps
        ops.raise_on_error(engine.runtime.device)
        out = {"prefill_tokens_per_s": round(tokens * 1000.0 / prefill_ms, 1), "prefill_ms": round(prefill_ms, 3),
               "decode_tokens_per_s": round(batch * 1000.0 / decode_ms, 1), "decode_ms": round(decode_ms, 4),
               "launches_per_decode_step": (ops.launches - launches) // steps}
        for r in requests:
            engine.cache.close(r.request_id)
        del engine
        torch.cuda.empty_cache()
        return out

    class Step:
        pass

    def step_of(lens, starts):
        st = Step()
        st.num_seqs, st.q_lens = len(lens), list(lens)
        cu = [0]
        for n in lens:
            cu.append(cu[-1] + n)
        st.num_tokens = cu[-1]
        st.cu_seqlens = torch.tensor(cu, dtype=torch.int32, device=dev)
        st.state_slots = torch.arange(len(lens), dtype=torch.int32, device=dev)
        st.positions = torch.tensor([s + i for s, n in zip(starts, lens) for i in range(n)], dtype=torch.int32, device=dev)
        st.seq_lens = torch.tensor([s + n for s, n in zip(starts, lens)], dtype=torch.int32, device=dev)
        st.seq_lens_host, st.max_q_len = [s + n for s, n in zip(starts, lens)], max(lens)
        st.max_seq_len = max(st.seq_lens_host)
        st.decode_only, st.workspace = all(n == 1 for n in lens), None
        return st


    def kernels(size: dict) -> dict:
        H, G, d, D = size["heads"], size["kv"], size["dim"], size["width"]
        window, run, cap = size["window"], size["run"], size["softcap"]
        E, top, F = size["experts"], size["top"], size["eff"]
        out = {}

        def note(name, ms, bytes_=None, flops=None):
            entry = {"us": round(ms * 1000.0, 2)}
            if bytes_ is not None:
                entry.update(gb_s=round(bytes_ / ms / 1e6, 1), frac_hbm=round(bytes_ / (ms / 1e3) / hbm, 4))
            if flops is not None:
                entry.update(tflops=round(flops / ms / 1e9, 2), frac_tensor=round(flops / (ms / 1e3) / flops_peak, 4))
            out[name] = entry

        for mode, lens, starts in (("prefill", [tokens], [0]), ("decode", [1] * batch, [context - 1] * batch)):
            st = step_of(lens, starts)
            T = sum(lens)
            page = 16
            pages = -(-st.max_seq_len // page)
            table = torch.arange(len(lens) * pages, dtype=torch.int32, device=dev).view(len(lens), pages)
            slots = torch.cat([table[i].long()[(st.positions[st.cu_seqlens[i]: st.cu_seqlens[i + 1]] // page).long()] * page
                               + st.positions[st.cu_seqlens[i]: st.cu_seqlens[i + 1]].long() % page for i in range(len(lens))])
            cache = (torch.randn(len(lens) * pages, 2, G, page, d, device=dev) * 0.3).to(bf)
            kv = KVView(cache, table, slots, page, window, True, KVSpec(((G, d), (G, d)), window))
            run_kv = KVView(cache, table, slots, page, None, True, KVSpec(((G, d), (G, d)), None, chunk=run))
            plain_kv = KVView(cache, table, slots, page, run, True, KVSpec.keys_and_values(G, d, run))
            st.token_ids = torch.randint(0, vocab, (T,), device=dev, dtype=torch.int32)
            # one norm over the whole projection, the rotation in neighbouring pairs over half a head, the cache
            # write; beside the norm of every head by itself with the rotation in split halves
            cols = (H + 2 * G) * d
            proj = (torch.randn(T, cols + H * d, device=dev) * 0.5).to(bf)  # q | k | v | gate
            inv = torch.tensor([100000.0 ** (-2.0 * i / (d // 2)) for i in range(d // 4)], device=dev)
            wq, wk, wh = torch.ones(H * d, device=dev), torch.ones(G * d, device=dev), torch.ones(d, device=dev)
            ms = timed(lambda: ops.qkv_prepare(proj, 0, H * d, (H + G) * d, H, d, None, wq, wk, 1e-5, inv, st.positions, kv, True,
                                               whole=True, interleaved=True), 20)
            note(f"qkv_prepare_whole_{mode}", ms, bytes_=T * cols * 4)
            ms = timed(lambda: ops.qkv_prepare(proj, 0, H * d, (H + G) * d, H, d, None, wh, wh, 1e-5, inv, st.positions, kv, True), 20)
            note(f"like:qkv_prepare_{mode}", ms, bytes_=T * cols * 4)
            # attention: the window with the gate on the heads' outputs; the runs with capped scores beside a
            # window as long as a run (which sees about twice the keys in a prompt: a run's queries see half a run
            # on average)
            q = (torch.randn(T, H, d, device=dev) * 0.3).to(bf)
            sink = torch.zeros(H, device=dev)
            reps = 5 if mode == "prefill" else 20

            def pairs(visible):
                return sum(visible(s + i) for s, n in zip(starts, lens) for i in range(n))

            in_window, in_run = pairs(lambda p: min(p + 1, window)), pairs(lambda p: p % run + 1)
            in_like = pairs(lambda p: min(p + 1, run))
            held_w = sum(min(s + n, window + n - 1) for s, n in zip(starts, lens))
            held_r = sum(min(s + n, (s % run) + n) for s, n in zip(starts, lens))
            held_l = sum(min(s + n, run + n - 1) for s, n in zip(starts, lens))
            moved = lambda held: held * 2 * G * d * 2 + 4 * T * H * d
            ms = timed(lambda: ops.paged_attention(q, kv, st, d ** -0.5, gate=proj, gate_col=cols, window=window), reps, 2)
            note(f"window_gate_attention_{mode}", ms, bytes_=moved(held_w) + 2 * T * H * d, flops=4 * in_window * H * d)
            dolutar_kv = KVView(cache, table, slots, page, window, True, KVSpec(((G, d), (G, d)), window, keep_first=size["keep"]))
            ms = timed(lambda: ops.paged_attention(q, dolutar_kv, st, d ** -0.5, sink=sink, window=window, keep_first=size["keep"]),
                       reps, 2)
            note(f"like:sink_window_attention_{mode}", ms, bytes_=moved(held_w), flops=4 * in_window * H * d)
            ms = timed(lambda: ops.paged_attention(q, run_kv, st, d ** -0.5, window=None, chunk=run, softcap=cap), reps, 2)
            note(f"run_capped_attention_{mode}", ms, bytes_=moved(held_r), flops=4 * in_run * H * d)
            ms = timed(lambda: ops.paged_attention(q, run_kv, st, d ** -0.5, window=None, chunk=run), reps, 2)
            note(f"run_attention_no_cap_{mode}", ms, bytes_=moved(held_r), flops=4 * in_run * H * d)
            ms = timed(lambda: ops.paged_attention(q, plain_kv, st, d ** -0.5), reps, 2)
            note(f"like:paged_attention_{mode}", ms, bytes_=moved(held_l), flops=4 * in_like * H * d)
            # the decayed linear attention (activations, recurrence, norm over all heads, gate) beside the gated delta
            # rule of equal heads and widths with the convolution ahead of it
            lcols = 2 * H * d + 2 * H * d  # q | k | v | gate
            lproj = (torch.randn(T, lcols, device=dev) * 0.5).to(bf)
            S_state = torch.zeros(len(lens) + 1, H, d, d, device=dev)
            decays = torch.full((H,), 0.99, device=dev)
            nw = torch.ones(H * d, device=dev)
            state_bytes = 2 * len(lens) * H * d * d * 4
            ms = timed(lambda: ops.lightning_attention(lproj, 0, H * d, 2 * H * d, 3 * H * d, H, d, d, decays, nw, 1e-5, S_state, st), 10)
            note(f"lightning_attention_{mode}", ms, bytes_=state_bytes + T * (4 * H * d * 2 + H * d * (4 + 4 + 2)),
                 flops=T * H * d * d * 2 * 2)
            C = 3 * H * d
            dproj = torch.randn(T, C + H, device=dev).to(bf)
            taps = torch.randn(C, 4, device=dev)
            conv_state = torch.zeros(len(lens) + 1, 3, C, device=dev)
            a, gate = torch.randn(T, H * d, device=dev).to(bf), torch.randn(T, H * d, device=dev).to(bf)
            A_log, dt_bias, nwh = torch.zeros(H, device=dev), torch.zeros(H * d, device=dev), torch.ones(d, device=dev)
            run_conv = lambda: ops.short_conv(dproj, 0, C, taps, conv_state, st, 2 * H * d, d, 1e-6, H * d, d ** -0.5,
                                              a, A_log, dt_bias, C, H)
            conv = run_conv()
            note(f"like:short_conv_{mode}", timed(run_conv, 20), bytes_=T * (C * (2 + 4) + H * d * (2 + 4)))
            S_state.zero_()
            ms = timed(lambda: ops.delta_rule(conv, C, H, H, d, d, dproj, 0, gate, nwh, 1e-5, S_state, conv_state, 4, st), 10)
            note(f"like:delta_rule_{mode}", ms, bytes_=state_bytes + T * ((C + H * d) * 4 + 2 * H * d * 2),
                 flops=T * H * d * d * 2 * 3)
            del S_state, lproj, dproj, conv
            # the relu-gated unit in its product, beside SwiGLU in the same product
            h = (torch.randn(T, D, device=dev) * 0.5).to(bf)
            gate_up = (torch.randn(2 * size["ff"], D, device=dev) * D ** -0.5).to(bf)
            dense = dict(bytes_=2 * size["ff"] * D * 2 + T * (D + size["ff"]) * 2, flops=2 * T * 2 * size["ff"] * D)
            note(f"linear_relu_glu_{mode}", timed(lambda: ops.linear_relu_glu(h, gate_up), 10), **dense)
            note(f"like:linear_swiglu_{mode}", timed(lambda: ops.linear_swiglu(h, gate_up), 10), **dense)
            del gate_up
            # experts chosen by the table (clamped units, equal weights) beside experts chosen by a router
            egu = (torch.randn(E, 2 * F, D, device=dev) * D ** -0.5).to(bf)
            edn = (torch.randn(E, D, F, device=dev) * F ** -0.5).to(bf)
            rows = [torch.randperm(E, generator=g)[:top] for _ in range(4096)]
            expert_table = torch.stack(rows).to(torch.int32).repeat(vocab // 4096, 1).to(dev).contiguous()
            router, correction = torch.randn(E, D, device=dev) * 0.05, torch.zeros(E, device=dev)
            counts = torch.zeros(E, dtype=torch.int32, device=dev)

            def route_table():
                counts.zero_()
                return ops.moe_route_table(st.token_ids, expert_table, E, counts)

            def route():
                counts.zero_()
                return ops.moe_route(h, router, correction, E, top, counts)

            note(f"moe_route_table_{mode}", timed(route_table, 20), bytes_=T * (4 + top * 12))
            note(f"like:moe_route_{mode}", timed(route, 20), bytes_=T * D * 2 + E * D * 4)
            used = E * (1.0 - (1.0 - top / E) ** T)  # experts that T tokens' choices touch, on average
            work = dict(bytes_=used * 3 * F * D * 2 + T * D * 4, flops=2 * T * top * 3 * F * D)
            ms = timed(lambda: ops.moe_experts(h, None, None, egu, edn, top, st, table=expert_table, token_ids=st.token_ids,
                                               alpha=1.702, limit=7.0), 10)
            note(f"table_experts_{mode}", ms, **work)
            ms = timed(lambda: ops.moe_experts(h, router, correction, egu, edn, top, st), 10)
            note(f"like:routed_experts_{mode}", ms, **work)
            del egu, edn
        ops.raise_on_error(dev)
        return out

    record = {"metric": "Bobarax beside Dolutar at equal sizes", "unit": "tokens/s", "dtype": "bf16",
              "data": "synthetic: seeded uniform-random token ids, random weights",
              "config": {"prefill_tokens": tokens, "decode_batch": batch, "decode_context": context, "vocab": vocab,
                         "peaks": peak_source}, "sizes": {}}
    for name in ([args.size] if args.size else list(BOBARAX_SIZES)):
        size = BOBARAX_SIZES[name]
        record["sizes"][name] = {"bobarax": whole_model(bobarax_config(size)), "dolutar": whole_model(dolutar_config(size)),
                                 "kernels": kernels(size), "layers": size["layers"]}
    return record

def narezen_config(size: dict) -> dict:
    """Layers in fours: attention whose values are its keys beside a channel-decayed state, rotated attention
    beside a retention, a gated recurrence over channels, and the first kind again; experts with a shared
    expert everywhere. The linear-attention sides have half the attention's heads, of the same widths."""
    H, G, d, D = size["heads"], size["kv"], size["dim"], size["width"]
    R = max(H // 2, 1)
    moe = {"kind": "moe", "expert": {"ff": size["eff"]}, "router": {"experts": size["experts"], "top": size["top"]},
           "shared": {"ff": size["eff"]}}
    layers = []
    for i in range(size["layers"]):
        kind = i % 4
        if kind in (0, 3):
            mixer = {"left": {"heads": H, "kv_heads": G, "dim": d, "vdim": d, "scale": 0.125},
                     "right": {"heads": R, "dim": d, "vdim": d, "tau": 16.0}, "left_scale": 1.2, "right_scale": 1.1}
            layers.append({"type": "parallel", "mixer": mixer, "mlp": moe})
        elif kind == 1:
            decay = [1.0 - 2.0 ** -(5 + 6 * h / max(R - 1, 1)) for h in range(R)]
            mixer = {"left": {"heads": H, "kv_heads": G, "dim": d, "vdim": d, "scale": d ** -0.5,
                              "rot": {"base": 100000.0, "dims": d // 2}},
                     "right": {"heads": R, "dim": d, "vdim": d, "decay": decay, "rot": {"base": 1e6, "dims": d}},
                     "left_scale": 1.2, "right_scale": 0.5}
            layers.append({"type": "parallel_2", "mixer": mixer, "mlp": moe})
        else:
            layers.append({"type": "rglru", "mixer": {"width": D, "blocks": H, "conv": 4}, "mlp": moe})
    return {"architecture": "Narezen", "vocab": DOLUTAR_VOCAB, "width": D, "embedding": {"scale": 1.0}, "norm": {"eps": 1e-5},
            "logit_softcap": 30.0, "layers": layers}


def run_narezen(args) -> dict:
    """Prefill (one prompt of --prefill-tokens) and decode (--batch requests ending at --context tokens)
    of Narezen and of Bobarax at equal sizes, then the new design's kernels alone, each beside the like
    kernel of Bobarax."""
    import torch

    from mlx_omnia_b200.engine.engine import Engine, EngineArgs
    from mlx_omnia_b200.engine.step import StepEntry
    from mlx_omnia_b200.kernels import ops
    from mlx_omnia_b200.parts.base import KVSpec, KVView

    measured, peak_source = peaks()
    hbm, flops_peak = measured["hbm_gbs"] * 1e9, measured["bf16_tflops"] * 1e12
    g = torch.Generator().manual_seed(SEED)
    steps, warmup, batch, context, tokens = args.steps, max(args.warmup, 3), args.batch, args.context, args.prefill_tokens
    dev, bf = torch.device("cuda:0"), torch.bfloat16
    vocab = DOLUTAR_VOCAB

    def timed(fn, count, warm=3):
        for _ in range(warm):
            fn()
        torch.cuda.synchronize()
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        for _ in range(count):
            fn()
        stop.record()
        torch.cuda.synchronize()
        return start.elapsed_time(stop) / count

    def whole_model(raw) -> dict:
        engine = Engine.from_random(raw, SEED, EngineArgs(dtype="bfloat16", page_size=16, max_requests=batch + 1,
                                                          cache_tokens=batch * (context + 16) + tokens + 16))
        times = []
        for index in range(warmup + 3):
            request = engine.cache.open(f"p{index}")
            ids = torch.randint(0, vocab, (tokens,), generator=g).tolist()
            torch.cuda.synchronize()
            start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record()
            engine.runner.run([StepEntry(request, ids, [tokens - 1])])
            stop.record()
            torch.cuda.synchronize()
            engine.cache.close(request.request_id)
            times.append(start.elapsed_time(stop))
        prefill_ms = statistics.median(times[warmup:])
        requests = [engine.cache.open(f"d{i}") for i in range(batch)]
        length = context - steps - warmup - 1
        for r in requests:
            engine.runner.run([StepEntry(r, torch.randint(0, vocab, (length,), generator=g).tolist(), [])])
        entries = lambda i: [StepEntry(r, [1 + i], [0]) for r in requests]
        for i in range(warmup):
            engine.runner.run(entries(i), copy=False)
        torch.cuda.synchronize()
        launches = ops.launches
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        for i in range(steps):
            engine.runner.run(entries(warmup + i), copy=False)
        stop.record()
        torch.cuda.synchronize()
        decode_ms = start.elapsed_time(stop) / steps
        ops.raise_on_error(engine.runtime.device)
        out = {"prefill_tokens_per_s": round(tokens * 1000.0 / prefill_ms, 1), "prefill_ms": round(prefill_ms, 3),
               "decode_tokens_per_s": round(batch * 1000.0 / decode_ms, 1), "decode_ms": round(decode_ms, 4),
               "launches_per_decode_step": (ops.launches - launches) // steps}
        for r in requests:
            engine.cache.close(r.request_id)
        del engine
        torch.cuda.empty_cache()
        return out

    class Step:
        pass

    def step_of(lens, starts):
        st = Step()
        st.num_seqs, st.q_lens = len(lens), list(lens)
        cu = [0]
        for n in lens:
            cu.append(cu[-1] + n)
        st.num_tokens = cu[-1]
        st.cu_seqlens = torch.tensor(cu, dtype=torch.int32, device=dev)
        st.state_slots = torch.arange(len(lens), dtype=torch.int32, device=dev)
        st.positions = torch.tensor([s + i for s, n in zip(starts, lens) for i in range(n)], dtype=torch.int32, device=dev)
        st.seq_lens = torch.tensor([s + n for s, n in zip(starts, lens)], dtype=torch.int32, device=dev)
        st.seq_lens_host, st.max_q_len = [s + n for s, n in zip(starts, lens)], max(lens)
        st.max_seq_len = max(st.seq_lens_host)
        st.decode_only, st.workspace = all(n == 1 for n in lens), None
        return st

    def kernels(size: dict) -> dict:
        H, G, d, D = size["heads"], size["kv"], size["dim"], size["width"]
        R = max(H // 2, 1)
        E, top, F = size["experts"], size["top"], size["eff"]
        out = {}

        def note(name, ms, bytes_=None, flops=None):
            entry = {"us": round(ms * 1000.0, 2)}
            if bytes_ is not None:
                entry.update(gb_s=round(bytes_ / ms / 1e6, 1), frac_hbm=round(bytes_ / (ms / 1e3) / hbm, 4))
            if flops is not None:
                entry.update(tflops=round(flops / ms / 1e9, 2), frac_tensor=round(flops / (ms / 1e3) / flops_peak, 4))
            out[name] = entry

        for mode, lens, starts in (("prefill", [tokens], [0]), ("decode", [1] * batch, [context - 1] * batch)):
            st = step_of(lens, starts)
            T = sum(lens)
            page = 16
            pages = -(-st.max_seq_len // page)
            table = torch.arange(len(lens) * pages, dtype=torch.int32, device=dev).view(len(lens), pages)
            slots = torch.cat([table[i].long()[(st.positions[st.cu_seqlens[i]: st.cu_seqlens[i + 1]] // page).long()] * page
                               + st.positions[st.cu_seqlens[i]: st.cu_seqlens[i + 1]].long() % page for i in range(len(lens))])
            cache = (torch.randn(len(lens) * pages, 2, G, page, d, device=dev) * 0.3).to(bf)
            kv = KVView(cache, table, slots, page, None, True, KVSpec(((G, d), (G, d))))
            # the input step of the attention whose values are its keys (weightless head norms, no rotation), beside
            # Bobarax's (one norm over the projection, rotation of neighbouring pairs)
            cols = (H + G) * d
            proj = (torch.randn(T, cols + G * d + H * d, device=dev) * 0.5).to(bf)
            ms = timed(lambda: ops.qkv_prepare(proj, 0, H * d, H * d, H, d, None, None, None, 1e-5, None, st.positions, kv, True), 20)
            note(f"qkv_prepare_keys_as_values_{mode}", ms, bytes_=T * (cols * 2 + (H + 2 * G) * d * 2))
            inv = torch.tensor([100000.0 ** (-2.0 * i / (d // 2)) for i in range(d // 4)], device=dev)
            wq, wk = torch.ones(H * d, device=dev), torch.ones(G * d, device=dev)
            ms = timed(lambda: ops.qkv_prepare(proj, 0, H * d, (H + G) * d, H, d, None, wq, wk, 1e-5, inv, st.positions, kv, True,
                                               whole=True, interleaved=True), 20)
            note(f"like:qkv_prepare_whole_{mode}", ms, bytes_=T * (H + 2 * G) * d * 4)
            # causal attention over every earlier position with a sink a head, beside Bobarax's windowed attention
            # with its gate (a window as long as the context sees the same keys)
            q = (torch.randn(T, H, d, device=dev) * 0.3).to(bf)
            sink = torch.zeros(H, device=dev)
            reps = 5 if mode == "prefill" else 20
            seen = sum(s + i + 1 for s, n in zip(starts, lens) for i in range(n))
            held = sum(s + n for s, n in zip(starts, lens))
            work = dict(bytes_=held * 2 * G * d * 2 + 4 * T * H * d, flops=4 * seen * H * d)
            ms = timed(lambda: ops.paged_attention(q, kv, st, 0.125, sink=sink), reps, 2)
            note(f"sink_attention_{mode}", ms, **work)
            wide = st.max_seq_len + 1
            wkv = KVView(cache, table, slots, page, wide, True, KVSpec(((G, d), (G, d)), wide))
            ms = timed(lambda: ops.paged_attention(q, wkv, st, d ** -0.5, gate=proj, gate_col=cols + G * d, window=wide), reps, 2)
            note(f"like:window_gate_attention_{mode}", ms, **work)
            # linear attention from a float32 state: a decay per key channel (with the input step that makes the
            # decays), a decay per head with rotated queries and keys, beside Bobarax's recurrence of equal heads
            lcols = 2 * R * d + 2 * R * d  # q | k | v | gate
            lproj = (torch.randn(T, lcols, device=dev) * 0.5).to(bf)
            z = torch.randn(T, R * d, device=dev) + 2.0  # the decays' logits come in float32
            zb = torch.zeros(R * d, device=dev)
            S_state = torch.zeros(len(lens) + 1, R, d, d, device=dev)
            decays = torch.full((R,), 0.99, device=dev)
            nw, nwh = torch.ones(R * d, device=dev), torch.ones(d, device=dev)
            rinv = torch.tensor([1e6 ** (-2.0 * i / d) for i in range(d // 2)], device=dev)
            state_bytes = 2 * len(lens) * R * d * d * 4
            moved = state_bytes + T * (4 * R * d * 2 + R * d * 2)
            ms = timed(lambda: ops.state_attention(lproj, 0, R * d, 2 * R * d, 3 * R * d, R, d, d, S_state, st, 1e-5,
                                                   decay_logits=z, decay_bias=zb, tau=16.0, q_scale=d ** -0.5, norm_weight=nwh), 10)
            note(f"channel_decay_attention_{mode}", ms, bytes_=moved + T * R * d * 2, flops=T * R * d * d * 2 * 2)
            S_state.zero_()
            ms = timed(lambda: ops.state_attention(lproj, 0, R * d, 2 * R * d, 3 * R * d, R, d, d, S_state, st, 1e-5,
                                                   decay=decays, inv_freq=rinv, k_scale=d ** -0.5), 10)
            note(f"retention_{mode}", ms, bytes_=moved, flops=T * R * d * d * 2 * 2)
            S_state.zero_()
            ms = timed(lambda: ops.lightning_attention(lproj, 0, R * d, 2 * R * d, 3 * R * d, R, d, d, decays, nw, 1e-5, S_state, st), 10)
            note(f"like:lightning_attention_{mode}", ms, bytes_=moved, flops=T * R * d * d * 2 * 2)
            del S_state, lproj
            # the gated recurrence over channels (convolution, block-diagonal gates, scan) of the model's width
            C, blocks, K = D, H, 4
            bw = C // blocks
            rproj = (torch.randn(T, 2 * C, device=dev) * 0.5).to(bf)
            xb, yb, cb, lam = (torch.zeros(C, device=dev) for _ in range(4))
            taps = torch.randn(C, K, device=dev) * 0.5
            gates = torch.randn(blocks, bw, 2 * bw, device=dev) * bw ** -0.5
            rb, ib = torch.zeros(C, device=dev), torch.zeros(C, device=dev)
            S1, conv_state = torch.zeros(len(lens) + 1, C, device=dev), torch.zeros(len(lens) + 1, K - 1, C, device=dev)
            ms = timed(lambda: ops.gated_channel_recurrence(rproj, 0, C, xb, yb, taps, cb, gates, rb, ib, lam, 8.0, S1, conv_state, st), 10)
            note(f"gated_channel_recurrence_{mode}", ms, bytes_=T * C * (2 * 2 + 2) + blocks * bw * 2 * bw * 4,
                 flops=2 * T * C * 2 * bw)
            del rproj
            # the two sides' sum beside the residual step (the like pass over a row)
            a, b = (torch.randn(T, D, device=dev).to(bf) for _ in range(2))
            note(f"scaled_sum_{mode}", timed(lambda: ops.scaled_sum(a, 1.2, b, 1.1), 20), bytes_=T * D * 6)
            x, w = torch.randn(T, D, device=dev), torch.ones(D, device=dev)
            note(f"like:add_rmsnorm_{mode}", timed(lambda: ops.add_rmsnorm(x, a, w, 1e-5, w, 1e-5), 20), bytes_=T * D * (4 + 4 + 2 + 2))
            # experts chosen by sigmoid scores and given the weighted token, with the shared expert, beside Bobarax's
            # experts chosen by a table
            h = (torch.randn(T, D, device=dev) * 0.5).to(bf)
            egu = (torch.randn(E, 2 * F, D, device=dev) * D ** -0.5).to(bf)
            edn = (torch.randn(E, D, F, device=dev) * F ** -0.5).to(bf)
            sgu, sdn = (torch.randn(2 * F, D, device=dev) * D ** -0.5).to(bf), (torch.randn(D, F, device=dev) * F ** -0.5).to(bf)
            rows = [torch.randperm(E, generator=g)[:top] for _ in range(4096)]
            expert_table = torch.stack(rows).to(torch.int32).repeat(vocab // 4096, 1).to(dev).contiguous()
            st.token_ids = torch.randint(0, vocab, (T,), device=dev, dtype=torch.int32)
            router = torch.randn(E, D, device=dev) * 0.05
            used = E * (1.0 - (1.0 - top / E) ** T)
            work = dict(bytes_=used * 3 * F * D * 2 + T * D * 4, flops=2 * T * top * 3 * F * D)
            ms = timed(lambda: ops.moe_experts(h, router, None, egu, edn, top, st, scoring="sigmoid", weigh="input"), 10)
            note(f"sigmoid_input_weighted_experts_{mode}", ms, **work)
            ms = timed(lambda: ops.moe_experts(h, None, None, egu, edn, top, st, table=expert_table, token_ids=st.token_ids,
                                               alpha=1.702, limit=7.0), 10)
            note(f"like:table_experts_{mode}", ms, **work)
            ms = timed(lambda: ops.linear(ops.linear_swiglu(h, sgu), sdn), 10)
            note(f"shared_expert_{mode}", ms, bytes_=3 * F * D * 2 + T * (2 * D + F) * 2, flops=2 * T * 3 * F * D)
            del egu, edn
        ops.raise_on_error(dev)
        return out

    record = {"metric": "Narezen beside Bobarax at equal sizes", "unit": "tokens/s", "dtype": "bf16",
              "data": "synthetic: seeded uniform-random token ids, random weights",
              "config": {"prefill_tokens": tokens, "decode_batch": batch, "decode_context": context, "vocab": vocab,
                         "peaks": peak_source}, "sizes": {}}
    for name in ([args.size] if args.size else list(BOBARAX_SIZES)):
        size = BOBARAX_SIZES[name]
        record["sizes"][name] = {"narezen": whole_model(narezen_config(size)), "bobarax": whole_model(bobarax_config(size)),
                                 "kernels": kernels(size), "layers": size["layers"]}
    return record


def main() -> int:
    parser = argparse.ArgumentParser()
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=64)
    parser.add_argument("--warmup", type=int, default=4)
    parser.add_argument("--impl", choices=["ours", "reference"], default="ours")
    parser.add_argument("--batch", type=int, default=8)
    parser.add_argument("--layers", type=int, default=0, help="run fewer layers than configs[2] has (named in config)")
    parser.add_argument("--timeline", action="store_true",
                        help="with --only decode|prefill and OMNIA_TIMELINE=1 in the environment: one step's "
                             "kernels with the time each takes in the stream, on stderr")
    parser.add_argument("--only", choices=["all", "decode", "prefill", "mixed", "portions", "sampling", "products", "elementwise", "fokalorn",
                                           "dolutar", "bobarax", "narezen"], default="all",
                        help="time one part only (small cases for profilers); prints a short record")
    parser.add_argument("--config", type=int, choices=sorted(CONFIGS), default=2,
                        help="with --only: the sizes of another benchmark configuration (3: 36 layers, hidden 4096, "
                             "32/8 heads, intermediate 12288, untied head, context 8192)")
    parser.add_argument("--context", type=int, default=0, help="tokens each request holds at the last timed step "
                                                               "(default: the configuration's own)")
    parser.add_argument("--prefill-tokens", type=int, default=PREFILL_TOKENS)
    parser.add_argument("--pool-tokens", type=int, default=0, help="at least this many tokens of cache pool (default: what the run needs)")
    parser.add_argument("--portion", type=int, default=256,
                        help="--only mixed: tokens of a prompt that run beside --batch decoding requests")
    parser.add_argument("--size", choices=sorted(FOKALORN_SIZES), default=None,
                        help="--only fokalorn, dolutar, bobarax or narezen: one size instead of all")
    args = parser.parse_args()
    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable":
                          "gabfssilva/mlx-omnia needs Apple's MLX (Metal) and Python >= 3.13; its offline install "
                          "fails here (no hatchling build backend, no mlx wheel for Linux)"}))
        return 0
    if args.gpus != 1:
        print("bench.py: this engine runs on one GPU; --gpus must be 1")
        return 2
    if args.config != 2 and args.only == "all":
        print("bench.py: the full record is of configuration 2; give --only decode|prefill|mixed with --config")
        return 2
    args.context = args.context or CONFIGS[args.config][1]
    if args.only == "fokalorn":
        print(json.dumps(run_fokalorn(args)))
        return 0
    if args.only == "bobarax":
        print(json.dumps(run_bobarax(args)))
        return 0
    if args.only == "narezen":
        print(json.dumps(run_narezen(args)))
        return 0
    if args.only == "dolutar":
        print(json.dumps(run_dolutar(args)))
        return 0
    if args.only == "all":
        args.warmup = max(args.warmup, 3)
    print(json.dumps(run(args)))
    return 0


if __name__ == "__main__":
    sys.exit(main())
