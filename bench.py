"""Decode and prefill throughput of the engine on one B200, with roofline fractions.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]

A "step" is one decode step.  The default run has the layer sizes of the
Qwen2.5-1.5B shape with random weights, a batch of 8 requests that each hold a
2,048-token prompt (context limit 4,096), bfloat16.  One JSON line is printed:
``value`` is decoded tokens per second timed on the device, ``e2e`` the same
through ``LLMEngine.generate_many`` (host token ids in, host token ids out),
``prefill`` the 2,048-token prompt step, ``roofline`` the decode step's bytes
(every weight once plus the cache of the live requests) over its time against
the measured copy bandwidth, ``points`` decoding at batch 1 and 64.
"""
from __future__ import annotations

import argparse
import gc
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

QWEN25_1P5B = {
    "architectures": ["Qwen2ForCausalLM"], "model_type": "qwen2",
    "vocab_size": 151936, "hidden_size": 1536, "intermediate_size": 8960, "num_hidden_layers": 28,
    "num_attention_heads": 12, "num_key_value_heads": 2, "max_position_embeddings": 4096,
    "rope_theta": 1000000.0, "rms_norm_eps": 1e-6, "attention_bias": True, "tie_word_embeddings": True,
}
# layer sizes of the larger models of the same architecture (the workloads of the `points` beyond the headline, and
# `--sizes 7b|14b --only decode|prefill`)
QWEN25_7B_SIZES = {"hidden_size": 3584, "intermediate_size": 18944, "num_attention_heads": 28, "num_key_value_heads": 4,
                   "vocab_size": 152064, "tie_word_embeddings": False}
QWEN25_14B_SIZES = {"hidden_size": 5120, "intermediate_size": 13824, "num_attention_heads": 40, "num_key_value_heads": 8,
                    "vocab_size": 152064, "tie_word_embeddings": False, "rms_norm_eps": 1e-5, "max_position_embeddings": 8192}
LAYERS_7B, LAYERS_14B, LAYERS_14B_RUN = 28, 48, 12
FULL_LAYERS = QWEN25_1P5B["num_hidden_layers"]
USE_GRAPHS = True     # --no-graphs: launch by launch (for profilers)
PROMPT = 2048
BLOCK = 16


def peaks() -> dict:
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    out = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}
    if os.path.exists(path):
        try:
            data = json.load(open(path))
            out["hbm_gbs"] = float(data.get("hbm_gbs", out["hbm_gbs"]))
            out["bf16_tflops"] = float(data.get("bf16_tflops", out["bf16_tflops"]))
            out["source"] = "measured"
        except Exception:
            pass
    return out


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while a region is timed."""

    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self) -> None:
        self.rows: list[list[str]] = []
        self._stop = threading.Event()
        self._thread = threading.Thread(target=self._loop, daemon=True)

    def _loop(self) -> None:
        while not self._stop.is_set():
            try:
                out = subprocess.run(["nvidia-smi", "-i", "0", f"--query-gpu={self.QUERY}",
                                      "--format=csv,noheader,nounits"], capture_output=True, text=True, timeout=5)
                if out.returncode == 0 and out.stdout.strip():
                    self.rows.append([item.strip() for item in out.stdout.strip().splitlines()[0].split(",")])
            except Exception:
                pass
            self._stop.wait(0.2)

    def __enter__(self):
        self._thread.start()
        return self

    def __exit__(self, *_):
        self._stop.set()
        self._thread.join(timeout=6)

    def summary(self) -> dict:
        clocks = sorted(int(row[0]) for row in self.rows if row and row[0].isdigit())
        maxima = [int(row[1]) for row in self.rows if len(row) > 1 and row[1].isdigit()]
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        reasons = [name for index, name in enumerate(names, start=2)
                   if any(len(row) > index and row[index].lower().startswith("active") for row in self.rows)]
        return {"sm_mhz": clocks[len(clocks) // 2] if clocks else None,
                "sm_max_mhz": max(maxima) if maxima else None, "reasons": reasons, "samples": len(self.rows)}


def build_model(layers: int, sizes: dict | None = None, dtype: str = "bfloat16"):
    """A model of the architecture with random weights made on the device: N(0, 0.02) matrices and biases,
    norm weights 1 + U(-0.1, 0.1), seed 0.  ``sizes`` overrides keys of the Qwen2.5-1.5B configuration."""
    import torch

    from llm_serving_engine_b200.config import load_config
    from llm_serving_engine_b200.models import DecoderModel, expected_tensors, parse_dtype
    from llm_serving_engine_b200.weights.loader import held_dtype

    compute = parse_dtype(dtype)
    config = dict(QWEN25_1P5B, **(sizes or {}), num_hidden_layers=layers)
    return build_from_config(config, compute), config


def build_from_config(config: dict, compute):
    """A model of any registered architecture with random weights made on the device (seed 0)."""
    import torch

    from llm_serving_engine_b200.config import load_config
    from llm_serving_engine_b200.models import DecoderModel, expected_tensors
    from llm_serving_engine_b200.weights.loader import held_dtype

    _, _, spec = load_config(config)
    generator = torch.Generator(device="cuda").manual_seed(0)
    weights = {}
    for name, tensor_spec in expected_tensors(spec).items():
        if tensor_spec.kind == "norm":
            tensor = 1.0 + (torch.rand(tensor_spec.shape, generator=generator, device="cuda") * 0.2 - 0.1)
        elif tensor_spec.kind == "positive":
            tensor = 0.1 + 0.9 * torch.rand(tensor_spec.shape, generator=generator, device="cuda")
        elif tensor_spec.kind == "mixing":
            tensor = torch.eye(*tensor_spec.shape, device="cuda") + (torch.rand(tensor_spec.shape, generator=generator, device="cuda") * 0.2 - 0.1)
        else:
            tensor = torch.randn(tensor_spec.shape, generator=generator, device="cuda") * 0.02
        weights[name] = tensor.to(held_dtype(tensor_spec, tensor.dtype, compute))
    return DecoderModel(spec, weights, compute, "cuda")


def time_decode(model, batch: int, steps: int, warmup: int, repeats: int = 1, prompt: int = 0):
    """Device time of decode steps at ``batch`` requests that hold ``prompt`` (default PROMPT) tokens each:
    ``repeats`` runs of ``steps`` steps, each between a pair of CUDA events.  Returns (median milliseconds a
    step, the bytes of keys and values a step of the median run reads, launches of one run, every run's
    milliseconds a step)."""
    import torch

    from llm_serving_engine_b200.cache.manager import CacheManager
    from llm_serving_engine_b200.config.runtime_config import CacheConfig
    from llm_serving_engine_b200.engine.step import StepEntry, StepRunner
    from llm_serving_engine_b200.kernels import library, ops
    from llm_serving_engine_b200.models import cache_requirements

    prompt = prompt or PROMPT
    context = model.spec.max_position_embeddings
    pages = batch * (context // BLOCK)
    cache = CacheManager(cache_requirements(model.spec), CacheConfig(BLOCK, pages), model.dtype, model.device,
                         context, num_state_slots=batch)
    runner = StepRunner(model, cache, max_tokens_per_step=max(PROMPT, batch), max_segments=batch,
                        use_graphs=USE_GRAPHS)
    generator = torch.Generator().manual_seed(1)
    ids = [f"d{index}" for index in range(batch)]
    runs = []
    with torch.inference_mode():
        for rid in ids:
            cache.create(rid)
            tokens = torch.randint(0, model.vocab_size, (prompt,), generator=generator).tolist()
            for lo in range(0, prompt, PROMPT):          # a long prompt goes in portions of PROMPT tokens
                runner.run([StepEntry(rid, tokens[lo:lo + PROMPT], [])])
        tokens = torch.randint(0, model.vocab_size, (batch,), generator=generator).tolist()
        out = torch.empty(batch, dtype=torch.int32, device=model.device)

        def one_step():
            logits = runner.run([StepEntry(rid, [token], [0]) for rid, token in zip(ids, tokens)])
            ops.argmax(logits, out)

        for _ in range(warmup):
            one_step()
        torch.cuda.synchronize()
        launches = 0
        for _ in range(repeats):
            before = library.launches() + runner.graph_kernel_launches
            start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record()
            for _ in range(steps):
                one_step()
            end.record()
            torch.cuda.synchronize()
            launches = library.launches() + runner.graph_kernel_launches - before
            runs.append(start.elapsed_time(end) / steps)
    order = sorted(range(repeats), key=lambda index: runs[index])
    median_run = order[repeats // 2]
    kv_bytes = batch * (prompt + warmup + median_run * steps + steps // 2) * cache.kv_bytes_per_token()
    cache.free_all()
    del runner, cache
    torch.cuda.empty_cache()
    return runs[median_run], kv_bytes, launches, runs


def time_prefill(model, repeats: int = 5):
    import torch

    from llm_serving_engine_b200.cache.manager import CacheManager
    from llm_serving_engine_b200.config.runtime_config import CacheConfig
    from llm_serving_engine_b200.engine.step import StepEntry, StepRunner
    from llm_serving_engine_b200.models import cache_requirements

    context = model.spec.max_position_embeddings
    cache = CacheManager(cache_requirements(model.spec), CacheConfig(BLOCK, context // BLOCK), model.dtype,
                         model.device, context, num_state_slots=1)
    runner = StepRunner(model, cache, max_tokens_per_step=PROMPT, max_segments=1)
    generator = torch.Generator().manual_seed(2)
    prompt = torch.randint(0, model.vocab_size, (PROMPT,), generator=generator).tolist()
    times = []
    with torch.inference_mode():
        for index in range(repeats + 2):
            cache.create("p")
            start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record()
            runner.run([StepEntry("p", prompt, [PROMPT - 1])])
            end.record()
            torch.cuda.synchronize()
            cache.free("p")
            if index >= 2:
                times.append(start.elapsed_time(end))
    times.sort()
    return times[len(times) // 2]


def prefill_flops(config: dict, layers: int, tokens: int) -> float:
    h, inter = config["hidden_size"], config["intermediate_size"]
    n_q, n_kv = config["num_attention_heads"], config["num_key_value_heads"]
    d = h // n_q
    linear = (n_q + 2 * n_kv) * d * h + n_q * d * h + 3 * inter * h
    attention = 4 * n_q * d * tokens * (tokens + 1) / 2
    return layers * (2.0 * tokens * linear + attention) + 2.0 * config["vocab_size"] * h


def time_e2e(model, batch: int, new_tokens: int):
    """Decode tokens per second through the Python entry point: host token ids in, host token ids
    out (``LLMEngine.generate_many`` with per-token callbacks).  The clock runs over the steps in
    which all ``batch`` requests decode together: from the moment the last of them has its first
    token to the moment the first of them ends."""
    import torch

    from llm_serving_engine_b200 import CacheConfig, GenerationConfig, LLMEngine, SchedulerConfig

    context = model.spec.max_position_embeddings
    engine = LLMEngine(model, None, cache_config=CacheConfig(BLOCK, batch * (context // BLOCK)),
                       scheduler_config=SchedulerConfig(max_batch_size=batch, max_tokens_per_step=max(PROMPT, batch)),
                       prefill_chunk_size=PROMPT)
    engine.warmup()
    generator = torch.Generator().manual_seed(3)
    prompts = [torch.randint(0, model.vocab_size, (PROMPT,), generator=generator).tolist() for _ in range(batch)]
    stamps: list[tuple[float, int]] = []

    def make_callback(index: int):
        def callback(_token: int) -> None:
            stamps.append((time.perf_counter(), index))
        return callback

    engine.generate_many(prompts, GenerationConfig(max_new_tokens=new_tokens + 2 * batch),
                         [make_callback(index) for index in range(batch)])
    torch.cuda.synchronize()
    counts = [0] * batch
    window_start = window_end = None
    for stamp, index in stamps:
        counts[index] += 1
        if window_start is None and min(counts) >= 1:
            window_start = stamp           # the last request got its first token
        if window_end is None and max(counts) >= new_tokens + 2 * batch:
            window_end = stamp             # the first request got its last token
    decoded = sum(1 for stamp, _ in stamps if window_start < stamp <= window_end)
    seconds = window_end - window_start
    h2d = engine.runner.last_h2d_bytes
    del engine
    torch.cuda.empty_cache()
    return decoded / max(seconds, 1e-9), h2d, 4 * batch, decoded // batch


REPEATS = 5     # runs of the timed decode region; the median is reported, the spread beside it


def time_mixed_traffic(model, requests: int = 32, seed: int = 0):
    """Continuous batching of ``requests`` requests through the Python entry point: prompt lengths log-normal
    (median 512, clipped to 64 .. 4,096), 128 to 512 output tokens each, all waiting at the start.  Returns
    (generated tokens a second over the whole run, generated tokens, prompt tokens, seconds)."""
    import torch

    from llm_serving_engine_b200 import CacheConfig, GenerationConfig, LLMEngine, SchedulerConfig
    from llm_serving_engine_b200.workload import ClippedLogNormal, TrafficProfile, make_traffic

    limit = model.spec.max_position_embeddings
    profile = TrafficProfile(requests=requests, arrival_rate=0.0, prompt=ClippedLogNormal(512, 1.0, 64, 4096),
                             output=ClippedLogNormal(256, 0.5, 128, 512), seed=seed,
                             vocabulary_size=model.vocab_size).fitted_to(model.vocab_size, limit)
    traffic = make_traffic(profile)
    engine = LLMEngine(model, None, cache_config=CacheConfig(BLOCK, requests * (limit // BLOCK)),
                       scheduler_config=SchedulerConfig(max_batch_size=requests, max_tokens_per_step=PROMPT),
                       prefill_chunk_size=PROMPT)
    engine.warmup()
    torch.cuda.synchronize()
    started = time.perf_counter()
    outputs = engine.generate_many([list(item.prompt_token_ids) for item in traffic],
                                   [GenerationConfig(max_new_tokens=item.max_new_tokens) for item in traffic])
    torch.cuda.synchronize()
    seconds = time.perf_counter() - started
    generated = sum(len(output) for output in outputs)
    del engine
    torch.cuda.empty_cache()
    return generated / seconds, generated, sum(len(item.prompt_token_ids) for item in traffic), seconds


def time_short_requests(model, batch: int, prompt: int = 128, new_tokens: int = 32, chunk: int = 32, repeats: int = 3):
    """The workload of the reference's committed T4 results (``artifacts/checkpoint3-t4.json``): ``batch`` prompts of
    ``prompt`` tokens, ``new_tokens`` generated tokens each, prompts fed in portions of ``chunk`` tokens, through the
    Python entry point.  Returns generated tokens a second over the whole run (the median of ``repeats`` runs)."""
    import torch

    from llm_serving_engine_b200 import CacheConfig, GenerationConfig, LLMEngine, SchedulerConfig

    engine = LLMEngine(model, None, cache_config=CacheConfig(BLOCK, batch * 16 + 16),
                       scheduler_config=SchedulerConfig(max_batch_size=batch, max_tokens_per_step=max(chunk, batch)),
                       prefill_chunk_size=chunk)
    engine.warmup()
    generator = torch.Generator().manual_seed(5)
    rates = []
    for _ in range(repeats + 1):     # the first run meets every size class for the first time
        prompts = [torch.randint(0, model.vocab_size, (prompt,), generator=generator).tolist() for _ in range(batch)]
        torch.cuda.synchronize()
        started = time.perf_counter()
        outputs = engine.generate_many(prompts, GenerationConfig(max_new_tokens=new_tokens))
        torch.cuda.synchronize()
        rates.append(sum(len(output) for output in outputs) / (time.perf_counter() - started))
    del engine
    torch.cuda.empty_cache()
    return sorted(rates[1:])[repeats // 2]


def time_chunks_beside_decoding(model, decoding: int = 8, prompt: int = 8192, chunk: int = 2048):
    """A ``prompt``-token prompt fed in ``chunk``-token portions beside ``decoding`` requests that decode (each
    holds ``chunk`` tokens): device milliseconds of each mixed step."""
    import torch

    from llm_serving_engine_b200.cache.manager import CacheManager
    from llm_serving_engine_b200.config.runtime_config import CacheConfig
    from llm_serving_engine_b200.engine.step import StepEntry, StepRunner
    from llm_serving_engine_b200.models import cache_requirements

    context = model.spec.max_position_embeddings
    cache = CacheManager(cache_requirements(model.spec), CacheConfig(BLOCK, (decoding + 1) * (context // BLOCK)), model.dtype,
                         model.device, context, num_state_slots=decoding + 1)
    runner = StepRunner(model, cache, max_tokens_per_step=chunk + decoding, max_segments=decoding + 1)
    generator = torch.Generator().manual_seed(4)
    times = []
    with torch.inference_mode():
        for index in range(decoding):
            cache.create(f"d{index}")
            runner.run([StepEntry(f"d{index}", torch.randint(0, model.vocab_size, (chunk,), generator=generator).tolist(), [])])
        for repeat in range(3):          # the first pass launches kernel by kernel, the second captures, the third replays
            cache.create("long")
            tokens = torch.randint(0, model.vocab_size, (prompt,), generator=generator).tolist()
            times = []
            for lo in range(0, prompt, chunk):
                entries = [StepEntry("long", tokens[lo:lo + chunk], [chunk - 1] if lo + chunk == prompt else [])]
                entries += [StepEntry(f"d{index}", [7], [0]) for index in range(decoding)]
                start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                start.record()
                runner.run(entries)
                end.record()
                torch.cuda.synchronize()
                times.append(start.elapsed_time(end))
            cache.free("long")
    cache.free_all()
    del runner, cache
    torch.cuda.empty_cache()
    return times


def kernel_table(batch: int, layers: int) -> dict | None:
    """Per kind of kernel, what one decode step spends in it: a child process loads the tuning variant of the
    library (its kernels stamp the device's clock) and prints the sums as JSON.  None when that fails."""
    try:
        done = subprocess.run([sys.executable, os.path.abspath(__file__), "--timeline", "1", "--timeline-json", "--batch", str(batch),
                               "--layers", str(layers)], capture_output=True, text=True, timeout=600)
        for line in reversed(done.stdout.strip().splitlines()):
            if line.startswith("{"):
                return json.loads(line)
    except Exception:
        pass
    return None


def other_points(args, peak: dict) -> tuple[dict, dict]:
    """The workloads beyond the headline: the float32 path, contexts of 30,000 keys, the Qwen2.5-7B sizes under mixed
    traffic, the Qwen2.5-14B sizes at context 8,192 (fewer layers than the model has: both numbers are in the point's
    name or note)."""
    import torch

    points, notes = {}, {}
    steps = max(args.steps // 4, 8)

    def attempt(name, work):
        try:
            work()
        except Exception as error:    # a point that fails is reported as missing, the headline stands
            points[name] = None
            notes[name] = f"{type(error).__name__}: {str(error)[:120]}"
        torch.cuda.empty_cache()

    def float32():
        model, _ = build_model(FULL_LAYERS, dtype="float32")
        ms, kv_bytes, _, _ = time_decode(model, 8, steps, 3)
        points["fp32_decode_b8"] = round(8 / (ms / 1e3), 1)
        notes["fp32_decode_b8"] = (f"true float32 path, 28 layers, {ms:.3f} ms a step, "
                                   f"{(model.weight_bytes_per_step() + kv_bytes) / (ms / 1e3) / 1e9 / peak['hbm_gbs']:.3f} of the copy bandwidth")

    def sizes_7b():
        model, _ = build_model(LAYERS_7B, QWEN25_7B_SIZES)
        rate, generated, prompts, seconds = time_mixed_traffic(model)
        points["7b_mixed32_output_tok_s"] = round(rate, 1)
        notes["7b_mixed32_output_tok_s"] = (f"Qwen2.5-7B sizes, 28 of 28 layers, 32 requests at once, {prompts} prompt and {generated} "
                                            f"generated tokens in {seconds:.2f} s through LLMEngine.generate_many")
        ms, kv_bytes, _, _ = time_decode(model, 8, steps, 3)
        points["7b_decode_b8"] = round(8 / (ms / 1e3), 1)
        notes["7b_decode_b8"] = f"{(model.weight_bytes_per_step() + kv_bytes) / (ms / 1e3) / 1e9 / peak['hbm_gbs']:.3f} of the copy bandwidth"

    def sizes_14b():
        model, _ = build_model(LAYERS_14B_RUN, QWEN25_14B_SIZES)
        for batch in (1, 8, 64):
            ms, kv_bytes, _, _ = time_decode(model, batch, steps, 3, prompt=8192 - 64)
            name = f"14b_{LAYERS_14B_RUN}of{LAYERS_14B}_layers_ctx8192_decode_b{batch}"
            points[name] = round(batch / (ms / 1e3), 1)
            notes[name] = f"{(model.weight_bytes_per_step() + kv_bytes) / (ms / 1e3) / 1e9 / peak['hbm_gbs']:.3f} of the copy bandwidth"
        times = time_chunks_beside_decoding(model)
        name = f"14b_{LAYERS_14B_RUN}of{LAYERS_14B}_layers_prefill8192_in_2048_chunks_beside_8_decoding_tok_s"
        points[name] = round(8192 / (sum(times) / 1e3), 1)
        notes[name] = "ms of the four mixed steps: " + ", ".join(f"{value:.2f}" for value in times)

    def long_contexts():
        model, _ = build_model(FULL_LAYERS, {"max_position_embeddings": 32768})
        for batch in (1, 8):
            ms, kv_bytes, _, _ = time_decode(model, batch, steps, 3, prompt=30000)
            name = f"ctx30000_decode_b{batch}"
            points[name] = round(batch / (ms / 1e3), 1)
            notes[name] = (f"the headline's model, {ms:.3f} ms a step, "
                           f"{(model.weight_bytes_per_step() + kv_bytes) / (ms / 1e3) / 1e9 / peak['hbm_gbs']:.3f} of the copy bandwidth")

    def short_requests():
        model, _ = build_model(FULL_LAYERS)
        published = {1: 18.84, 8: 128.61}    # the reference's own Tesla T4 results for this workload (the real Qwen2.5-1.5B, float16)
        for batch in (1, 8):
            rate = time_short_requests(model, batch)
            name = f"128x32_chunk32_b{batch}_output_tok_s"
            points[name] = round(rate, 1)
            notes[name] = (f"{batch} prompts of 128 tokens, 32 generated tokens each, portions of 32, through generate_many; the "
                           f"reference publishes {published[batch]} on a Tesla T4 for this workload (no B200 figure exists)")

    attempt("fp32_decode_b8", float32)
    attempt("128x32_chunk32", short_requests)
    attempt("ctx30000_decode", long_contexts)
    attempt("7b_mixed32_output_tok_s", sizes_7b)
    attempt("14b", sizes_14b)
    return points, notes


def run_ours(args) -> dict:
    import torch

    import __graft_entry__
    __graft_entry__.build()
    torch.cuda.set_device(0)
    layers = args.layers or FULL_LAYERS
    sizes = {"7b": QWEN25_7B_SIZES, "14b": QWEN25_14B_SIZES}.get(args.sizes)
    model, config = build_model(layers, sizes, dtype=args.dtype if args.only != "all" else "bfloat16")
    peak = peaks()
    weight_bytes = model.weight_bytes_per_step()
    batch = args.batch

    if args.only == "decode":     # a short run of one part, for profilers; prints no bench line
        ms, kv_bytes, _, _ = time_decode(model, batch, args.steps, args.warmup)
        return {"only": "decode", "batch": batch, "layers": layers, "ms_per_step": round(ms, 4),
                "gb_per_s": round((weight_bytes + kv_bytes) / (ms / 1000) / 1e9, 1)}
    if args.only == "prefill":
        ms = time_prefill(model, repeats=max(1, args.steps))
        return {"only": "prefill", "layers": layers, "ms": round(ms, 4),
                "tflops": round(prefill_flops(config, layers, PROMPT) / (ms / 1000) / 1e12, 1)}
    with ClockSampler() as clocks:
        ms, kv_bytes, launches, runs = time_decode(model, batch, args.steps, args.warmup, repeats=REPEATS)
    value = batch / (ms / 1e3)
    achieved = (weight_bytes + kv_bytes) / (ms / 1e3) / 1e9

    prefill_ms = time_prefill(model)
    flops = prefill_flops(config, layers, PROMPT)
    points, fractions = {}, {}
    for point_batch in (1, 64):
        point_ms, point_kv, _, _ = time_decode(model, point_batch, max(args.steps // 2, 8), args.warmup, repeats=3)
        points[f"decode_b{point_batch}"] = round(point_batch / (point_ms / 1e3), 1)
        fractions[f"decode_b{point_batch}"] = round((weight_bytes + point_kv) / (point_ms / 1e3) / 1e9 / peak["hbm_gbs"], 4)
    e2e_value, h2d, d2h, _ = time_e2e(model, batch, max(args.steps, 16))
    del model
    torch.cuda.empty_cache()
    more, notes = ({}, {}) if args.quick else other_points(args, peak)
    points.update(more)
    kernels = None if args.quick else kernel_table(batch, layers)

    return {
        "metric": "decode tok/s at batch 8 (Qwen2.5-1.5B shape, 2,048-token prompts)",
        "value": round(value, 1), "unit": "tokens/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": round(ms, 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic (random weights, uniform random token ids)", "impl": "ours",
        "config": bench_config(config, layers, batch),
        "repeats": {"count": REPEATS, "ms_per_step": [round(run, 4) for run in runs], "reported": "median",
                    "spread": round((max(runs) - min(runs)) / ms, 4)},
        "prefill": {"value": round(PROMPT / (prefill_ms / 1e3), 1), "tokens": PROMPT, "ms": round(prefill_ms, 3),
                    "frac": round(flops / (prefill_ms / 1e3) / (peak["bf16_tflops"] * 1e12), 4)},
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": peak["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / peak["hbm_gbs"], 4), "peaks": peak["source"]},
        "points": points, "points_roofline_frac": fractions, "points_notes": notes,
        "kernels": kernels,
        "e2e": {"value": round(e2e_value, 1), "unit": "tokens/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                "pipeline": "one decode step in flight: every step copies its metadata from pinned host memory and its "
                            "tokens to the host; the tokens feed the next step on the device"},
        "gpu_launches": launches,
        "clocks": clocks.summary(),
    }


# -- another design beside the closest existing model ------------------------------------------
# Layer sizes that resemble real models of the kind (heads of 128, a latent of 512 with a rotated part of 64,
# query latents of three quarters of the width, feed-forwards of four widths), six layers in the order
# [latent, lightning, latent reading layer 0's cache, latent_2, latent_2, lightning]; feed-forwards where a latent
# layer stands, none behind the lightning layers; four residual streams.
GIVELIX_SIZES = {
    "w2048": dict(width=2048, heads=16, ff=8192, q_rank=1536),
    "w4096": dict(width=4096, heads=32, ff=16384, q_rank=3072),
}


def givelix_config(width: int, heads: int, ff: int, q_rank: int, vocab: int = 32768, context: int = 4096) -> dict:
    rot = {"base": 500000.0, "dims": 64}
    scaled = dict(rot, scaling={"factor": 4.0, "original": 1024, "fast": 32.0, "slow": 1.0})
    mlp = {"kind": "dense", "ff": ff}
    first = {"heads": heads, "dim": 128, "rot_dim": 64, "vdim": 128, "kv_rank": 512, "q_rank": q_rank,
             "scale": 192 ** -0.5, "rot": rot}
    second = {"heads": heads, "dim": 128, "rot_dim": 64, "vdim": 128, "kv_rank": 512, "scale": 192 ** -0.5, "rot": scaled}
    linear = {"heads": heads, "dim": 128, "vdim": 128, "decay": [1.0 - 2.0 ** -(3 + 5 * h / max(heads - 1, 1)) for h in range(heads)]}
    layers = [{"type": "latent_attention", "mixer": first, "mlp": mlp},
              {"type": "lightning", "mixer": linear, "mlp": None},
              {"type": "latent_attention", "mixer": dict(first, kv_from=0), "mlp": mlp},
              {"type": "latent_attention_2", "mixer": second, "mlp": mlp},
              {"type": "latent_attention_2", "mixer": second, "mlp": mlp},
              {"type": "lightning", "mixer": linear, "mlp": None}]
    return {"architecture": "Givelix", "vocab": vocab, "width": width, "layers": layers, "norm": {"eps": 1e-5},
            "residual_mult": 0.3, "streams": 4, "logit_scale": 0.5, "max_position_embeddings": context}


# Fororax at layer sizes that resemble real models of the kind: heads of 128 in groups of eight, six layers in the order
# [attention_2, attention, attention reading layer 1's keys and values, attention_2, attention_2, attention], every layer
# with a mixture of eight experts and two identity experts of which a token uses two, beside a shared expert; an expert
# and the shared one are a third of the Qwen2 feed-forward each, so that a token's work equals the dense layer's.
FORORAX_SIZES = {
    "w2048": dict(width=2048, heads=16, ff=8192),
    "w4096": dict(width=4096, heads=32, ff=16384),
}
# Tufevik at layer sizes that resemble real models of the kind: six layers, matrix-memory layers and layers with an
# attention and a selective scan side by side in turn; heads of 128 (the attention's in groups of eight, half of a head
# rotated, four taps), a scan of as many channels as the model is wide with sixteen states a channel and a step-size
# rank of a sixteenth of the width; dense feed-forwards and mixtures of eight experts of half the dense size of which a
# token uses two in turn, so that a token's feed-forward work equals the dense layer's.
TUFEVIK_SIZES = {
    "w2048": dict(width=2048, heads=16, ff=8192),
    "w4096": dict(width=4096, heads=32, ff=16384),
}
# Sebudra at layer sizes that resemble real models of the kind: six layers in the order [side by side, sigmoid attention,
# matrix memory with channel decays, side by side, sigmoid attention, matrix memory]; attention heads of 128 in groups of
# eight (the windowed one over 512 keys, half of a head rotated with stretched frequencies); a state-space scan of as
# many channels as the model is wide in heads of 64 with 128 state rows and two groups, four taps; a matrix memory with
# heads of 64 key channels and 128 values and a decay map of rank 32; dense feed-forwards and mixtures of eight ungated
# experts in four groups (two kept) of half the dense size of which a token uses two, beside a shared expert of the same
# size, so that a token's feed-forward work equals the gated dense layer's.  The closest existing model is Tufevik (an
# attention and a scan side by side, a matrix memory, mixtures of experts): it is measured beside it at equal size.
SEBUDRA_SIZES = {
    "w2048": dict(width=2048, heads=16, ff=8192),
    "w4096": dict(width=4096, heads=32, ff=16384),
}
DESIGN_SIZES = {"givelix": GIVELIX_SIZES, "fororax": FORORAX_SIZES, "tufevik": TUFEVIK_SIZES, "sebudra": SEBUDRA_SIZES}


def fororax_config(width: int, heads: int, ff: int, vocab: int = 32768, context: int = 4096) -> dict:
    expert_ff = (ff // 3) // 64 * 64
    mlp = {"kind": "moe", "router": {"experts": 8, "identity": 2, "top": 2}, "expert": {"ff": expert_ff, "limit": 7.0},
           "shared": {"ff": ff - 2 * expert_ff, "limit": 7.0}}
    mixer = {"heads": heads, "kv_heads": max(2, heads // 8), "dim": 128, "vdim": 128, "scale": 128 ** -0.5}
    kinds = ["attention_2", "attention", "attention", "attention_2", "attention_2", "attention"]
    layers = [{"type": kind, "mixer": dict(mixer, kv_from=1) if index == 2 else dict(mixer), "mlp": mlp}
              for index, kind in enumerate(kinds)]
    return {"architecture": "Fororax", "vocab": vocab, "width": width, "max_positions": context, "layers": layers,
            "norm": {"eps": 1e-6}, "postln_alpha": 2.0, "embedding": {"scale": 1.0}, "logit_softcap": 30.0}


def tufevik_config(width: int, heads: int, ff: int, vocab: int = 32768, context: int = 4096) -> dict:
    dense = {"kind": "dense", "ff": ff}
    mixture = {"kind": "moe", "router": {"experts": 8, "top": 2}, "expert": {"ff": ff // 2}}
    memory = {"heads": heads, "dim": 128, "vdim": 128, "gate_cap": 12.0}
    left = {"heads": heads, "kv_heads": max(2, heads // 8), "dim": 128, "vdim": 128, "conv": 4, "scale": 128 ** -0.5,
            "rot": {"base": 500000.0, "dims": 64, "scaling": {"factor": 4.0, "original": 2048, "fast": 16.0, "slow": 1.0}}}
    right = {"inner": width, "state": 16, "dt_rank": width // 16, "conv": 4}
    side_by_side = {"left": left, "right": right, "left_scale": 0.5, "right_scale": 0.5}
    layers = [{"type": "mlstm", "mixer": memory, "mlp": dense}, {"type": "parallel", "mixer": side_by_side, "mlp": mixture},
              {"type": "mlstm", "mixer": memory, "mlp": mixture}, {"type": "parallel", "mixer": side_by_side, "mlp": dense},
              {"type": "mlstm", "mixer": memory, "mlp": dense}, {"type": "parallel", "mixer": side_by_side, "mlp": mixture}]
    return {"architecture": "Tufevik", "vocab": vocab, "width": width, "layers": layers, "norm": {"eps": 1e-6},
            "embedding": {"scale": 1.0}, "max_position_embeddings": context}


def sebudra_config(width: int, heads: int, ff: int, vocab: int = 32768, context: int = 4096) -> dict:
    dense = {"kind": "dense", "ff": ff, "limit": 7.0}
    mixture = {"kind": "moe", "router": {"experts": 8, "top": 2, "scale": 2.5, "groups": {"count": 4, "keep": 2}},
               "expert": {"ff": ff // 2}, "shared": {"ff": ff // 2}}
    kv_heads = max(2, heads // 8)
    left = {"heads": heads, "kv_heads": kv_heads, "dim": 128, "vdim": 128, "scale": 128 ** -0.5, "mask": {"size": 512},
            "rot": {"base": 1000000.0, "dims": 64, "scaling": {"factor": 8.0, "original": 2048, "fast": 16.0, "slow": 1.0}}}
    right = {"heads": width // 64, "vdim": 64, "state": 128, "groups": 2, "conv": 4, "norm_groups": 2}
    side_by_side = {"left": left, "right": right, "left_scale": 0.5, "right_scale": 0.5}
    attention = {"heads": heads, "kv_heads": kv_heads, "dim": 128, "vdim": 128, "scale": 128 ** -0.5, "softcap": 50.0,
                 "rot": {"base": 1000000.0, "dims": 128}}
    memory = {"heads": heads, "dim": 64, "vdim": 128, "tau": 8.0, "rank": 32}
    layers = [{"type": "parallel", "mixer": side_by_side, "mlp": dense}, {"type": "attention", "mixer": attention, "mlp": mixture},
              {"type": "gla", "mixer": memory, "mlp": mixture}, {"type": "parallel", "mixer": side_by_side, "mlp": dense},
              {"type": "attention", "mixer": attention, "mlp": dense}, {"type": "gla", "mixer": memory, "mlp": mixture}]
    return {"architecture": "Sebudra", "vocab": vocab, "width": width, "layers": layers, "norm": {"eps": 1e-6},
            "embedding": {"scale": 1.0}, "max_position_embeddings": context}


def kernel_times(run, repeats: int = 3) -> dict:
    """Device microseconds per kernel name (a mean over ``repeats`` calls of ``run``), from the profiler's records."""
    import torch
    from torch.profiler import ProfilerActivity, profile

    from llm_serving_engine_b200.kernels import library

    # Without programmatic dependent launch for the measurement: a kernel that is launched early spends the tail of
    # the kernel before it waiting, and the profiler would count that wait as its own time.
    library.load().lse_set_pdl(0)
    try:
        run()
        torch.cuda.synchronize()
        with profile(activities=[ProfilerActivity.CUDA]) as prof:
            for _ in range(repeats):
                run()
            torch.cuda.synchronize()
    finally:
        library.load().lse_set_pdl(0 if os.environ.get("LSE_PDL", "1") == "0" else 1)
    table = {}
    for event in prof.key_averages():
        total = getattr(event, "device_time_total", None) or getattr(event, "cuda_time_total", 0)
        if total:
            name = event.key.replace("(anonymous namespace)::", "").replace("void ", "").split("(")[0].split("<")[0]
            entry = table.setdefault(name, [0, 0.0])
            entry[0] += event.count / repeats
            entry[1] += total / repeats
    return {name: {"launches": round(count, 1), "us": round(us, 1)} for name, (count, us) in
            sorted(table.items(), key=lambda item: -item[1][1])}


def run_design(args) -> dict:
    """``--design NAME``: prefill and decode throughput of the named design at two layer sizes beside a Qwen2
    model of equal width, depth, heads and feed-forward, and the device time of every kernel of a prompt step and a
    decode step, with roofline fractions of the kernels that the two designs do not share."""
    import torch

    import __graft_entry__
    __graft_entry__.build()
    torch.cuda.set_device(0)
    from llm_serving_engine_b200.cache.manager import CacheManager
    from llm_serving_engine_b200.config.runtime_config import CacheConfig
    from llm_serving_engine_b200.engine.step import StepEntry, StepRunner
    from llm_serving_engine_b200.models import cache_requirements, parse_dtype

    peak = peaks()
    fma_tflops = 2 * 128 * torch.cuda.get_device_properties(0).multi_processor_count * 1.965e9 / 1e12   # float32 FMA pipe
    design = args.design
    make_config = {"givelix": givelix_config, "fororax": fororax_config, "tufevik": tufevik_config,
                   "sebudra": sebudra_config}[design]
    rooflines = {"givelix": design_rooflines, "fororax": fororax_rooflines, "tufevik": tufevik_rooflines,
                 "sebudra": sebudra_rooflines}[design]
    # designs that are set beside another model than Qwen2 as well: (label, config maker)
    beside = {"sebudra": [("tufevik_equal_size", tufevik_config)]}.get(design, [])
    batch, out = args.batch, {"design": design, "peaks": dict(peak, fp32_fma_tflops=round(fma_tflops, 1)), "sizes": {}}
    names = [args.design_size] if args.design_size else list(DESIGN_SIZES[design])
    with ClockSampler() as clocks:
        for size in names:
            shape = DESIGN_SIZES[design][size]
            qwen = dict(QWEN25_1P5B, vocab_size=32768, hidden_size=shape["width"], intermediate_size=shape["ff"],
                        num_hidden_layers=6, num_attention_heads=shape["heads"], num_key_value_heads=max(2, shape["heads"] // 8))
            entry = {}
            models = [(design, make_config(**shape))] + [(label, make(**shape)) for label, make in beside]
            for label, config in models + [("qwen2_equal_size", qwen)]:
                model = build_from_config(config, parse_dtype("bfloat16"))
                prefill_ms = time_prefill(model)
                decode_ms, _, _, _ = time_decode(model, batch, args.steps, max(args.warmup, 3), repeats=3)
                row = {"prefill_tokens_per_s": round(PROMPT / (prefill_ms / 1e3), 1), "prefill_ms": round(prefill_ms, 3),
                       "decode_tokens_per_s": round(batch / (decode_ms / 1e3), 1), "decode_ms_per_step": round(decode_ms, 4),
                       "weight_gb": round(model.weight_bytes_per_step() / 1e9, 3)}
                if not args.quick:
                    context = model.spec.max_position_embeddings
                    cache = CacheManager(cache_requirements(model.spec), CacheConfig(BLOCK, (batch + 1) * (context // BLOCK)),
                                         model.dtype, model.device, context, num_state_slots=batch + 1)
                    runner = StepRunner(model, cache, max_tokens_per_step=PROMPT, max_segments=batch, use_graphs=False)
                    generator = torch.Generator().manual_seed(4)
                    prompt = torch.randint(0, model.vocab_size, (PROMPT,), generator=generator).tolist()

                    def prompt_step():
                        cache.create("p")
                        runner.run([StepEntry("p", prompt, [PROMPT - 1])])
                        cache.free("p")

                    with torch.inference_mode():
                        row["prefill_kernels"] = kernel_times(prompt_step)
                        ids = [f"d{index}" for index in range(batch)]
                        for rid in ids:
                            cache.create(rid)
                            runner.run([StepEntry(rid, prompt, [])])
                        row["decode_kernels"] = kernel_times(lambda: runner.run([StepEntry(rid, [1], [0]) for rid in ids]))
                    cache.free_all()
                    del runner, cache
                entry[label] = row
                del model
                gc.collect()
                torch.cuda.empty_cache()
            if not args.quick:
                entry["roofline"] = rooflines(shape, entry, batch, peak, fma_tflops)
            out["sizes"][size] = entry
    out["clocks"] = clocks.summary()
    out["how"] = ("random weights, bfloat16, one 2,048-token prompt per prefill, decode at batch %d over 2,048-token "
                  "contexts; kernel times from the profiler's device records, launch by launch" % batch)
    return out


def design_rooflines(shape: dict, entry: dict, batch: int, peak: dict, fma_tflops: float) -> dict:
    """Fraction of its roofline that each kernel which the two designs do not share reaches: the slower of
    (bytes it must move / measured copy bandwidth) and (floating-point work / the peak of the pipe it runs on)
    over its measured time.  Givelix's attention scores, weights and recurrent state are float32 by the design's
    own rule, so its attention and scan kernels are set against the float32 FMA pipe; Qwen2's attention against
    the measured bfloat16 tensor throughput."""
    heads, width, tokens = shape["heads"], shape["width"], PROMPT
    kv_heads = max(2, heads // 8)
    bandwidth, tensor = peak["hbm_gbs"] * 1e9, peak["bf16_tflops"] * 1e12
    fma = fma_tflops * 1e12

    def frac(kernels: dict, key: str, launches_of_work: float, bytes_each: float, flops_each: float, pipe: float):
        found = [(name, value) for name, value in kernels.items() if key in name]
        if not found:
            return None
        us = sum(value["us"] for _, value in found)
        count = sum(value["launches"] for _, value in found)
        bound = max(bytes_each / bandwidth, flops_each / pipe) * launches_of_work
        return {"us": round(us, 1), "launches": count, "bound_us": round(bound * 1e6, 2), "frac": round(bound * 1e6 / us, 4)}

    pairs = tokens * (tokens + 1) / 2
    g, q = entry["givelix"], entry["qwen2_equal_size"]
    out = {"prefill": {}, "decode": {}}
    # prompt step: per launch of a layer
    out["prefill"]["givelix latent_attention (tensor cores)"] = frac(
        g["prefill_kernels"], "latent_attention_mma", 4, tokens * heads * (576 + 512) * 2, 2 * pairs * heads * (576 + 512), tensor)
    out["prefill"]["givelix linear_attention scan + carry (float32 FMA)"] = frac(
        g["prefill_kernels"], "linear_attention", 2, tokens * heads * 128 * 3 * 2 + tokens * heads * 128 * 4,
        tokens * heads * 128 * 128 * 2 * 4, fma)       # two passes of (state update + its use), a multiply-add each
    out["prefill"]["givelix streams_update_rmsnorm"] = frac(
        g["prefill_kernels"], "streams_update_rmsnorm", 11, tokens * width * (4 * 4 * 2 + 2 + 2), 0, fma)
    out["prefill"]["qwen2 attention (tcgen05)"] = frac(
        q["prefill_kernels"], "attn_", 6, tokens * (heads + 2 * kv_heads) * 128 * 2 * 2, 4 * pairs * heads * 128, tensor)
    out["prefill"]["qwen2 add_rmsnorm"] = frac(
        q["prefill_kernels"], "add_rmsnorm", 13, tokens * width * (4 * 2 + 2 + 2), 0, fma)
    # decode step at `batch` requests over 2,048-token contexts
    out["decode"]["givelix latent_attention (tensor cores, chunks + merge)"] = frac(
        g["decode_kernels"], "latent_attention_m", 4, batch * tokens * 576 * 2, 2 * batch * tokens * heads * (576 + 512), tensor)
    out["decode"]["givelix linear_attention scan"] = frac(
        g["decode_kernels"], "linear_attention", 2, batch * heads * 128 * 128 * 4 * 2, batch * heads * 128 * 128 * 4, fma)
    out["decode"]["givelix per-head products (few rows)"] = frac(
        g["decode_kernels"], "head_gemm", 8, heads * 128 * 512 * 2, 2 * batch * heads * 128 * 512, fma)
    out["decode"]["givelix streams_update_rmsnorm"] = frac(
        g["decode_kernels"], "streams_update_rmsnorm", 11, batch * width * (4 * 4 * 2 + 4 + 2), 0, fma)
    out["decode"]["qwen2 attention (mma.sync, split keys)"] = frac(
        q["decode_kernels"], "attn_", 6, batch * tokens * 2 * kv_heads * 128 * 2, 4 * batch * tokens * heads * 128, tensor)
    out["decode"]["qwen2 add_rmsnorm"] = frac(
        q["decode_kernels"], "add_rmsnorm", 13, batch * width * (4 * 2 + 4 + 2), 0, fma)
    return out


def fororax_rooflines(shape: dict, entry: dict, batch: int, peak: dict, fma_tflops: float) -> dict:
    """As :func:`design_rooflines`, for Fororax beside Qwen2: the attention kernels (bfloat16 tensor work; attention_2
    applies every head's weights to the values of every key/value head, which is counted as the work it is), the
    mixture's products against the dense feed-forward's (the work of the experts that a token uses; bytes of the experts
    that a step touches), and the row-wise kernels (bytes)."""
    heads, width, tokens = shape["heads"], shape["width"], PROMPT
    kv_heads = max(2, heads // 8)
    config = fororax_config(**shape)
    mlp = config["layers"][0]["mlp"]
    expert_ff, shared_ff, experts, top = mlp["expert"]["ff"], mlp["shared"]["ff"], mlp["router"]["experts"], mlp["router"]["top"]
    bandwidth, tensor, fma = peak["hbm_gbs"] * 1e9, peak["bf16_tflops"] * 1e12, fma_tflops * 1e12

    def frac(kernels: dict, keys, launches_of_work: float, bytes_each: float, flops_each: float, pipe: float):
        keys = (keys,) if isinstance(keys, str) else keys
        found = [(name, value) for name, value in kernels.items() if any(key in name for key in keys)]
        if not found:
            return None
        us = sum(value["us"] for _, value in found)
        count = sum(value["launches"] for _, value in found)
        bound = max(bytes_each / bandwidth, flops_each / pipe) * launches_of_work
        return {"us": round(us, 1), "launches": count, "bound_us": round(bound * 1e6, 2), "frac": round(bound * 1e6 / us, 4)}

    pairs = tokens * (tokens + 1) / 2
    f, q = entry["fororax"], entry["qwen2_equal_size"]
    out = {"prefill": {}, "decode": {}}
    # attention: 3 layers of each kind; attention_2 takes Q K^T and P V once per key/value head's values
    qkv_bytes = tokens * (heads + 2 * kv_heads) * 128 * 2 * 2
    work = 4 * pairs * heads * 128
    out["prefill"]["fororax attention (tcgen05; 3 layers with the penalty, 3 with sink and all groups' values)"] = frac(
        f["prefill_kernels"], ("attention_scored_mma", "attn_prefill_tc"), 3 + 3 * kv_heads, qkv_bytes, work, tensor)
    out["prefill"]["qwen2 attention (tcgen05)"] = frac(q["prefill_kernels"], "attn_", 6, qkv_bytes, work, tensor)
    # feed-forward products: Qwen2's are library products of [tokens, width] x [3 ff, width]; the mixture's are the
    # grouped products over the chosen experts' rows and the shared expert's plain products
    dense_flops = 2 * tokens * width * 3 * shape["ff"]
    moe_flops = 2 * tokens * width * 3 * (top * (experts / (experts + 2.0)) * expert_ff + shared_ff)   # a fifth of the choices are identity experts
    out["prefill"]["fororax mixture products (grouped + shared, library)"] = {
        "work_gflop_a_layer": round(moe_flops / 1e9, 1), "note": "library kernels: see the kernel table for their time"}
    out["prefill"]["qwen2 feed-forward products (library)"] = {"work_gflop_a_layer": round(dense_flops / 1e9, 1)}
    out["prefill"]["fororax rows of the mixture (route, place, gather, activation, combine)"] = frac(
        f["prefill_kernels"], ("moe_",), 6, tokens * width * 2 * (1 + 2 * top) + tokens * (top * expert_ff + shared_ff) * 2 * 3 + tokens * width * 4 * 2, 0, fma)
    out["prefill"]["fororax scaled_add_rmsnorm"] = frac(
        f["prefill_kernels"], "scaled_add_rmsnorm", 12, tokens * width * (4 * 2 + 4 + 2), 0, fma)
    out["prefill"]["fororax head_norm_kv_write"] = frac(
        f["prefill_kernels"], "head_norm_kv_write", 6, tokens * (heads + 2 * kv_heads) * 128 * 2 * 2, 0, fma)
    out["prefill"]["qwen2 add_rmsnorm"] = frac(q["prefill_kernels"], "add_rmsnorm", 13, tokens * width * (4 * 2 + 2 + 2), 0, fma)
    out["prefill"]["qwen2 rope_kv_write"] = frac(q["prefill_kernels"], "rope_kv_write", 6, tokens * (heads + 2 * kv_heads) * 128 * 2 * 2, 0, fma)
    # decode step at `batch` requests over 2,048-token contexts
    kv_bytes = batch * tokens * 2 * kv_heads * 128 * 2
    out["decode"]["fororax attention (mma.sync, chunks + merge)"] = frac(
        f["decode_kernels"], ("attention_scored",), 3 + 3 * kv_heads, kv_bytes, 4 * batch * tokens * heads * 128, tensor)
    out["decode"]["qwen2 attention (mma.sync, split keys)"] = frac(
        q["decode_kernels"], "attn_", 6, kv_bytes, 4 * batch * tokens * heads * 128, tensor)
    out["decode"]["fororax scaled_add_rmsnorm"] = frac(f["decode_kernels"], "scaled_add_rmsnorm", 12, batch * width * (4 * 2 + 4 + 2), 0, fma)
    out["decode"]["fororax rows of the mixture (route, activation)"] = frac(
        f["decode_kernels"], ("moe_",), 6, (experts + 3) * width * 2 + batch * (experts * expert_ff + shared_ff) * 2 * 3, 0, fma)
    out["decode"]["qwen2 add_rmsnorm"] = frac(q["decode_kernels"], "add_rmsnorm", 13, batch * width * (4 * 2 + 4 + 2), 0, fma)
    return out


def tufevik_rooflines(shape: dict, entry: dict, batch: int, peak: dict, fma_tflops: float) -> dict:
    """As :func:`design_rooflines`, for Tufevik beside Qwen2.  The matrix memory's scan and the selective scan keep
    float32 states by the design's own rule and are set against the float32 FMA pipe (an exponential counted as one
    operation) or the bytes they move, whichever is slower; the attention against the measured bfloat16 tensor
    throughput; the row-wise kernels (tanh norms, convolutions with norms and rotation, gates, read-outs) against the
    bytes they move."""
    heads, width, tokens = shape["heads"], shape["width"], PROMPT
    kv_heads = max(2, heads // 8)
    config = tufevik_config(**shape)
    right = config["layers"][1]["mixer"]["right"]
    inner, states, rank = right["inner"], right["state"], right["dt_rank"]
    mixture = config["layers"][1]["mlp"]
    experts, top, expert_ff = mixture["router"]["experts"], mixture["router"]["top"], mixture["expert"]["ff"]
    bandwidth, tensor, fma = peak["hbm_gbs"] * 1e9, peak["bf16_tflops"] * 1e12, fma_tflops * 1e12

    def frac(kernels: dict, keys, launches_of_work: float, bytes_each: float, flops_each: float, pipe: float):
        keys = (keys,) if isinstance(keys, str) else keys
        found = [(name, value) for name, value in kernels.items() if any(key in name for key in keys)]
        if not found:
            return None
        us = sum(value["us"] for _, value in found)
        count = sum(value["launches"] for _, value in found)
        bound = max(bytes_each / bandwidth, flops_each / pipe) * launches_of_work
        return {"us": round(us, 1), "launches": count, "bound_us": round(bound * 1e6, 2), "frac": round(bound * 1e6 / us, 4)}

    pairs = tokens * (tokens + 1) / 2
    t, q = entry["tufevik"], entry["qwen2_equal_size"]
    out = {"prefill": {}, "decode": {}}
    channels = (heads + 2 * kv_heads) * 128
    # prompt step: three matrix-memory layers, three layers with attention and scan side by side
    out["prefill"]["tufevik matrix memory scan + carry (float32 FMA)"] = frac(
        t["prefill_kernels"], "linear_attention", 3, tokens * heads * (128 * 3 * 4 + 129 * 4), tokens * heads * 128 * 129 * 2 * 4, fma)
    out["prefill"]["tufevik matrix memory gates + read-out"] = frac(
        t["prefill_kernels"], ("mlstm_gates", "mlstm_readout"), 3, tokens * heads * (129 * 4 + 128 * 4 + 128 * 2 + 5 * 4), 0, fma)
    out["prefill"]["tufevik selective scan (float32 FMA)"] = frac(
        t["prefill_kernels"], "selective_scan", 3, tokens * inner * (2 + 4 + 4 + 2) + tokens * 2 * states * 4,
        tokens * inner * states * 6, fma)
    out["prefill"]["tufevik step sizes + convolution of the scan's inputs"] = frac(
        t["prefill_kernels"], ("ssm_step_sizes", "short_conv_act"), 3, tokens * inner * (4 + 2) + tokens * inner * 4,
        2 * tokens * inner * rank, fma)
    out["prefill"]["tufevik attention (3 layers)"] = frac(
        t["prefill_kernels"], ("attention_scored", "attn_prefill_tc"), 3, tokens * channels * 2 * 2, 4 * pairs * heads * 128, tensor)
    out["prefill"]["tufevik conv_qk_norm_rope (+ head gates)"] = frac(
        t["prefill_kernels"], ("conv_qk_norm_rope", "head_gate_scale"), 3, tokens * channels * (4 + 2) + tokens * heads * 128 * 4, 0, fma)
    out["prefill"]["tufevik tanh_norm"] = frac(t["prefill_kernels"], "tanh_norm", 13, tokens * width * (4 * 2 + 4 + 2), 0, fma)
    out["prefill"]["tufevik rows of the mixture (route, place, gather, activation, combine)"] = frac(
        t["prefill_kernels"], ("moe_",), 3, tokens * width * 2 * (1 + 2 * top) + tokens * top * expert_ff * 2 * 3 + tokens * width * 4 * 2, 0, fma)
    out["prefill"]["qwen2 attention (tcgen05)"] = frac(
        q["prefill_kernels"], "attn_", 6, tokens * channels * 2 * 2, 4 * pairs * heads * 128, tensor)
    out["prefill"]["qwen2 add_rmsnorm"] = frac(q["prefill_kernels"], "add_rmsnorm", 13, tokens * width * (4 * 2 + 2 + 2), 0, fma)
    out["prefill"]["qwen2 rope_kv_write"] = frac(q["prefill_kernels"], "rope_kv_write", 6, tokens * channels * 2 * 2, 0, fma)
    # decode step at `batch` requests over 2,048-token contexts: the states are read and written once a token
    kv_bytes = batch * tokens * 2 * kv_heads * 128 * 2
    out["decode"]["tufevik matrix memory scan"] = frac(
        t["decode_kernels"], "linear_attention", 3, batch * heads * 128 * 129 * 4 * 2, batch * heads * 128 * 129 * 4, fma)
    out["decode"]["tufevik matrix memory gates + read-out"] = frac(
        t["decode_kernels"], ("mlstm_gates", "mlstm_readout"), 3, batch * heads * (129 * 4 + 128 * 4 + 128 * 2), 0, fma)
    out["decode"]["tufevik selective scan"] = frac(
        t["decode_kernels"], "selective_scan", 3, batch * inner * states * 4 * 2 + inner * states * 4, batch * inner * states * 6, fma)
    out["decode"]["tufevik step sizes + convolution of the scan's inputs"] = frac(
        t["decode_kernels"], ("ssm_step_sizes", "short_conv_act"), 3, inner * rank * 4 + batch * inner * 4 * 4, 2 * batch * inner * rank, fma)
    out["decode"]["tufevik attention (chunks + merge)"] = frac(
        t["decode_kernels"], ("attention_scored",), 3, kv_bytes, 4 * batch * tokens * heads * 128, tensor)
    out["decode"]["tufevik conv_qk_norm_rope (+ head gates)"] = frac(
        t["decode_kernels"], ("conv_qk_norm_rope", "head_gate_scale"), 3, batch * channels * 4 * 5, 0, fma)
    out["decode"]["tufevik tanh_norm"] = frac(t["decode_kernels"], "tanh_norm", 13, batch * width * (4 * 2 + 4 + 2), 0, fma)
    out["decode"]["tufevik rows of the mixture (route, activation)"] = frac(
        t["decode_kernels"], ("moe_",), 3, (experts + 1) * width * 2 + batch * experts * expert_ff * 2 * 3, 0, fma)
    out["decode"]["qwen2 attention (mma.sync, split keys)"] = frac(
        q["decode_kernels"], "attn_", 6, kv_bytes, 4 * batch * tokens * heads * 128, tensor)
    out["decode"]["qwen2 add_rmsnorm"] = frac(q["decode_kernels"], "add_rmsnorm", 13, batch * width * (4 * 2 + 4 + 2), 0, fma)
    return out


def sebudra_rooflines(shape: dict, entry: dict, batch: int, peak: dict, fma_tflops: float) -> dict:
    """As :func:`design_rooflines`, for Sebudra beside Tufevik (the closest existing model) at equal size: every kind of
    kernel that the two designs do not share, each against the slower of the bytes it must move and the operations it
    must do (scans and row-wise kernels against the float32 FMA pipe, attention against the measured bfloat16 tensor
    throughput)."""
    heads, width, tokens = shape["heads"], shape["width"], PROMPT
    kv_heads = max(2, heads // 8)
    config = sebudra_config(**shape)
    left, right = config["layers"][0]["mixer"]["left"], config["layers"][0]["mixer"]["right"]
    memory, mixture = config["layers"][2]["mixer"], config["layers"][1]["mlp"]
    window, ssm_heads, states, ssm_vdim = left["mask"]["size"], right["heads"], right["state"], right["vdim"]
    inner, groups = ssm_heads * ssm_vdim, right["groups"]
    conv_channels = inner + 2 * groups * states
    gla_heads, gla_dim, gla_vdim = memory["heads"], memory["dim"], memory["vdim"]
    experts, top, expert_ff = mixture["router"]["experts"], mixture["router"]["top"], mixture["expert"]["ff"]
    bandwidth, tensor, fma = peak["hbm_gbs"] * 1e9, peak["bf16_tflops"] * 1e12, fma_tflops * 1e12

    def frac(kernels: dict, keys, launches_of_work: float, bytes_each: float, flops_each: float, pipe: float, without=()):
        keys = (keys,) if isinstance(keys, str) else keys
        found = [(name, value) for name, value in kernels.items()
                 if any(key in name for key in keys) and not any(key in name for key in without)]
        if not found:
            return None
        us = sum(value["us"] for _, value in found)
        count = sum(value["launches"] for _, value in found)
        bound = max(bytes_each / bandwidth, flops_each / pipe) * launches_of_work
        return {"us": round(us, 1), "launches": count, "bound_us": round(bound * 1e6, 2), "frac": round(bound * 1e6 / us, 4)}

    pairs = tokens * (tokens + 1) / 2
    windowed_pairs = tokens * window - window * (window - 1) / 2
    s, t = entry["sebudra"], entry["tufevik_equal_size"]
    out = {"prefill": {}, "decode": {}}
    channels = (heads + 2 * kv_heads) * 128
    # Both of Sebudra's scans run in the engine's matrix-memory scan kernel: two state-space layers (state rows x head
    # channels per head) and two channel-decay memories.
    ssm_state, gla_state = ssm_heads * states * ssm_vdim, gla_heads * gla_dim * gla_vdim
    scan_bytes = 2 * (tokens * (conv_channels * 2 + inner * 4)) + 2 * (tokens * gla_heads * (2 * gla_dim + 2 * gla_vdim) * 4)
    scan_flops = 2 * tokens * ssm_state * 4 * 2 + 2 * tokens * gla_state * 4 * 2       # two passes of update and read-out
    out["prefill"]["sebudra scans (state space + channel decay, float32 FMA)"] = frac(
        s["prefill_kernels"], "linear_attention", 1, scan_bytes, scan_flops, fma)
    out["prefill"]["sebudra gates, decays, gated norms in parts"] = frac(
        s["prefill_kernels"], ("ssd_gates", "sigmoid_power", "gated_group_rmsnorm"), 1,
        2 * tokens * (inner * (4 + 4 + 2 + 2)) + 2 * tokens * gla_heads * (gla_dim * 8 + gla_vdim * 10), 0, fma)
    out["prefill"]["sebudra convolution of the scan's inputs"] = frac(
        s["prefill_kernels"], ("short_conv",), 2, tokens * conv_channels * (4 + 2), 0, fma)
    attention_flops = 2 * 4 * windowed_pairs * heads * 128 + 2 * 4 * pairs * heads * 128
    out["prefill"]["sebudra attention (2 windowed + 2 sigmoid layers)"] = frac(
        s["prefill_kernels"], ("attention_scored", "attn_prefill_tc"), 1, 4 * tokens * channels * 2 * 2, attention_flops, tensor)
    out["prefill"]["sebudra head norm + rotation + page write (+ branch scale)"] = frac(
        s["prefill_kernels"], ("head_norm_rope", "head_gate_scale"), 4, tokens * channels * (4 + 2) + tokens * heads * 128 * 4, 0, fma)
    out["prefill"]["sebudra add_rmsnorm (a stack of two branch outputs)"] = frac(
        s["prefill_kernels"], "add_rmsnorm", 7, tokens * width * (4 * 2 + 2 * 4 + 2), 0, fma)
    out["prefill"]["sebudra rows of the mixture (route, place, gather, activation, combine)"] = frac(
        s["prefill_kernels"], ("moe_",), 3, tokens * width * 2 * (1 + 2 * top) + tokens * top * expert_ff * 2 * 2 + tokens * width * 4 * 2, 0, fma)
    out["prefill"]["tufevik scans (matrix memory + selective, float32 FMA)"] = frac(
        t["prefill_kernels"], ("linear_attention", "selective_scan"), 1,
        3 * tokens * heads * (128 * 3 * 4 + 129 * 4) + 3 * (tokens * width * 12 + tokens * 2 * 16 * 4),
        3 * tokens * heads * 128 * 129 * 2 * 4 + 3 * tokens * width * 16 * 6, fma)
    out["prefill"]["tufevik attention (3 layers)"] = frac(
        t["prefill_kernels"], ("attention_scored", "attn_prefill_tc"), 3, tokens * channels * 2 * 2, 4 * pairs * heads * 128, tensor)
    out["prefill"]["tufevik conv_qk_norm_rope (+ head gates)"] = frac(
        t["prefill_kernels"], ("conv_qk_norm_rope", "head_gate_scale"), 3, tokens * channels * (4 + 2) + tokens * heads * 128 * 4, 0, fma)
    out["prefill"]["tufevik tanh_norm"] = frac(t["prefill_kernels"], "tanh_norm", 13, tokens * width * (4 * 2 + 4 + 2), 0, fma)
    out["prefill"]["tufevik rows of the mixture"] = frac(
        t["prefill_kernels"], ("moe_",), 3, tokens * width * 2 * (1 + 2 * top) + tokens * top * expert_ff * 2 * 3 + tokens * width * 4 * 2, 0, fma)
    out["prefill"] = {key: value for key, value in out["prefill"].items() if value is not None}
    # decode step at `batch` requests over 2,048-token contexts: the states are read and written once a token
    full_kv = batch * tokens * 2 * kv_heads * 128 * 2
    window_kv = batch * window * 2 * kv_heads * 128 * 2
    out["decode"]["sebudra scans (4 layers)"] = frac(
        s["decode_kernels"], "linear_attention", 1, batch * (2 * ssm_state + 2 * gla_state) * 4 * 2,
        batch * (2 * ssm_state + 2 * gla_state) * 4, fma)
    out["decode"]["sebudra gates, decays, gated norms in parts, convolution"] = frac(
        s["decode_kernels"], ("ssd_gates", "sigmoid_power", "gated_group_rmsnorm", "short_conv"), 1,
        2 * batch * (inner * 16 + conv_channels * 4 * 5) + 2 * batch * gla_heads * (gla_dim * 8 + gla_vdim * 10), 0, fma)
    out["decode"]["sebudra attention (2 windowed + 2 sigmoid layers, chunks + merge)"] = frac(
        s["decode_kernels"], ("attention_scored",), 1, 2 * full_kv + 2 * window_kv,
        2 * 4 * batch * (tokens + window) * heads * 128, tensor)
    out["decode"]["sebudra head norm + rotation + page write (+ branch scale)"] = frac(
        s["decode_kernels"], ("head_norm_rope", "head_gate_scale"), 4, batch * channels * 4 * 5, 0, fma)
    out["decode"]["sebudra add_rmsnorm"] = frac(s["decode_kernels"], "add_rmsnorm", 7, batch * width * (4 * 2 + 4 * 4 + 2), 0, fma)
    out["decode"]["sebudra rows of the mixture (route, activation)"] = frac(
        s["decode_kernels"], ("moe_",), 3, (experts + 1) * width * 2 + batch * (experts + 1) * expert_ff * 2 * 2, 0, fma)
    out["decode"]["tufevik scans"] = frac(
        t["decode_kernels"], ("linear_attention", "selective_scan"), 1,
        3 * batch * heads * 128 * 129 * 4 * 2 + 3 * (batch * width * 16 * 4 * 2),
        3 * batch * heads * 128 * 129 * 4 + 3 * batch * width * 16 * 6, fma)
    out["decode"]["tufevik attention (chunks + merge)"] = frac(
        t["decode_kernels"], ("attention_scored",), 3, full_kv, 4 * batch * tokens * heads * 128, tensor)
    out["decode"]["tufevik conv_qk_norm_rope (+ head gates)"] = frac(
        t["decode_kernels"], ("conv_qk_norm_rope", "head_gate_scale"), 3, batch * channels * 4 * 5, 0, fma)
    out["decode"]["tufevik tanh_norm"] = frac(t["decode_kernels"], "tanh_norm", 13, batch * width * (4 * 2 + 4 + 2), 0, fma)
    out["decode"]["tufevik rows of the mixture (route, activation)"] = frac(
        t["decode_kernels"], ("moe_",), 3, (experts + 1) * width * 2 + batch * experts * expert_ff * 2 * 3, 0, fma)
    out["decode"] = {key: value for key, value in out["decode"].items() if value is not None}
    return out


def bench_config(config: dict, layers: int, batch: int) -> dict:
    """The ``config`` of the bench line: every size, flat; the same dict in both arms."""
    return {
        "model": "Qwen2.5-1.5B shape", "layers": layers, "layers_full": FULL_LAYERS, "hidden": config["hidden_size"],
        "heads": config["num_attention_heads"], "kv_heads": config["num_key_value_heads"],
        "head_dim": config["hidden_size"] // config["num_attention_heads"],
        "intermediate": config["intermediate_size"], "vocab": config["vocab_size"], "tied": True,
        "global_batch": batch, "seq_len": PROMPT, "context": config["max_position_embeddings"],
        "kv_block": BLOCK, "parallelism": "single GPU", "l2": "inputs larger than L2 (weights 3 GB per step)",
    }


# -- the reference arm -----------------------------------------------------------------------
REFERENCE_DIR = os.path.join(ROOT, "baseline", "_ref")


def install_reference() -> str:
    """Put the unmodified reference into ``baseline/_ref`` (once, where its source tree is at hand) and
    return how.  The offline ``pip install`` is tried first; the reference's build backend (hatchling) is
    not in the wheelhouse, and its wheel is nothing but the pure-Python package ``src/llmserve``
    (``pyproject.toml``: ``packages = ["src/llmserve"]``), so a plain copy of that folder is the install."""
    import shutil

    if os.path.exists(os.path.join(REFERENCE_DIR, "llmserve", "engine.py")):
        return "present"
    source = os.environ.get("LLMSERVE_REFERENCE", "/root/reference")
    if not os.path.isdir(os.path.join(source, "src", "llmserve")):
        return ""
    os.makedirs(REFERENCE_DIR, exist_ok=True)
    pip = subprocess.run([sys.executable, "-m", "pip", "install", "--no-index", "--no-build-isolation", "--no-deps",
                          "--find-links", "/opt/wheelhouse", "--target", REFERENCE_DIR, source],
                         capture_output=True, text=True)
    if pip.returncode == 0 and os.path.exists(os.path.join(REFERENCE_DIR, "llmserve", "engine.py")):
        return "pip"
    shutil.copytree(os.path.join(source, "src", "llmserve"), os.path.join(REFERENCE_DIR, "llmserve"),
                    ignore=shutil.ignore_patterns("__pycache__"), dirs_exist_ok=True)
    return "copy of src/llmserve (pip: no hatchling in the wheelhouse)"


def run_reference(args) -> dict:
    """The same metric and configuration through the UNMODIFIED reference: ``llmserve`` imported from
    ``baseline/_ref`` and nowhere else, its ``Transformer(ModelConfig(...))`` with its own random
    initialisation (``src/llmserve/cli.py:39-41``), its stock CUDA path (float16, ``cli.py:34``; Triton paged
    attention, ``engine.py:140-155``) and its public API (``LLMEngine.generate`` with per-token callbacks,
    ``engine.py:188-221``).  Nothing of this repository's package is imported.

    Device time per step comes from the CUDA event pairs that the reference records around every
    iteration when ``collect_iteration_metrics`` is on (the list behind its ``iteration_stats``,
    ``engine.py:246-254,358-370,438-458``): the decode iterations in which all requests decode together,
    the first ``--warmup`` of them left out, the next ``--steps`` taken.  ``e2e`` is measured from the
    callbacks' time stamps over the same iterations, as in this repository's own arm."""
    how = install_reference()
    if not how:
        return {"impl": "reference", "unavailable": "baseline/_ref holds no install of the reference and its source tree is not at hand"}
    sys.path.insert(0, REFERENCE_DIR)
    try:
        import asyncio

        import torch
        import llmserve
        from llmserve.config import CacheConfig, ModelConfig, SchedulerConfig
        from llmserve.engine import GenerationConfig, LLMEngine
        from llmserve.model import Transformer
        from llmserve.tokenizer import ByteTokenizer
        from llmserve.triton_kernels import is_triton_paged_attention_available
    except Exception as error:   # a missing dependency of the reference
        return {"impl": "reference", "unavailable": f"the reference does not import: {type(error).__name__}: {error}"}
    if not os.path.abspath(llmserve.__file__).startswith(REFERENCE_DIR):
        return {"impl": "reference", "unavailable": f"llmserve was imported from {llmserve.__file__}, not from baseline/_ref"}
    if "llm_serving_engine_b200" in sys.modules:
        raise RuntimeError("the reference arm must not load this repository's package")
    torch.cuda.set_device(0)
    device = torch.device("cuda")
    layers = args.layers or FULL_LAYERS
    config = dict(QWEN25_1P5B, num_hidden_layers=layers)
    peak = peaks()
    torch.manual_seed(0)
    model = Transformer(ModelConfig.from_dict(config))
    model = model.to(device=device, dtype=torch.float16).eval()
    backend = "triton" if is_triton_paged_attention_available(device) else "pytorch"
    if backend == "pytorch":
        return {"impl": "reference", "unavailable": "the reference's Triton paged attention reports itself unavailable on this GPU; "
                "its PyTorch block loop walks every (row, block) pair in Python: hours for 2,048-token prompts"}
    weight_bytes = sum(p.numel() * p.element_size() for p in model.parameters())   # tied head counted once
    kv_bytes_per_token = 2 * layers * config["num_key_value_heads"] * (config["hidden_size"] // config["num_attention_heads"]) * 2

    def make_engine(batch: int):
        return LLMEngine(model, ByteTokenizer(), cache_config=CacheConfig(BLOCK, batch * (config["max_position_embeddings"] // BLOCK)),
                         scheduler_config=SchedulerConfig(max_batch_size=batch, max_tokens_per_step=max(PROMPT, batch)),
                         paged_attention_backend=backend, prefill_chunk_size=PROMPT, collect_iteration_metrics=True,
                         device=device, dtype=torch.float16)

    def decode_run(batch: int, steps: int, warmup: int, inference_mode: bool = False):
        """(device ms per full-batch decode step, its median, end-to-end tokens/s over the same steps, the
        engine's stats).  ``inference_mode``: the driver wraps the run in ``torch.inference_mode()``."""
        with torch.inference_mode(inference_mode):
            return _decode_run(batch, steps, warmup)

    def _decode_run(batch: int, steps: int, warmup: int):
        engine = make_engine(batch)
        generator = torch.Generator().manual_seed(3)
        prompts = [torch.randint(0, config["vocab_size"], (PROMPT,), generator=generator).tolist() for _ in range(batch)]
        new_tokens = warmup + steps + 2 * batch + 2
        stamps: list[tuple[float, int]] = []

        def make_callback(index: int):
            def callback(_token: int) -> None:
                stamps.append((time.perf_counter(), index))
            return callback

        async def drive():
            try:
                await asyncio.gather(*[engine.generate(prompt, GenerationConfig(max_new_tokens=new_tokens, temperature=0.0),
                                                       make_callback(index)) for index, prompt in enumerate(prompts)])
                return engine.iteration_stats
            finally:
                await engine.close()

        stats = asyncio.run(drive())
        # iterations in which all requests decode together: from the one after the last request got its first
        # token to the one in which the first request got its last token; one stamp per request and iteration
        counts = [0] * batch
        first_full = last_full = None
        for position, (_, index) in enumerate(stamps):
            counts[index] += 1
            if first_full is None and min(counts) >= 1:
                first_full = position + 1
            if last_full is None and max(counts) >= new_tokens:
                last_full = position        # the first request's last token opens an iteration: that one is left out
        full = stamps[first_full:last_full]
        iterations = len(full) // batch
        if len(full) != iterations * batch or iterations < warmup + steps:
            raise RuntimeError(f"reference arm: {len(full)} stamps in the all-decoding window do not make {warmup + steps} steps of {batch}")
        events = engine._iteration_cuda_events["decode"][:iterations]    # the list behind iteration_stats
        times = sorted(a.elapsed_time(b) for a, b in events[warmup:warmup + steps])
        ms = sum(times) / len(times)
        begin = full[warmup * batch - 1][0] if warmup else stamps[first_full - 1][0]
        end = full[(warmup + steps) * batch - 1][0]
        e2e = steps * batch / max(end - begin, 1e-9)
        del engine, drive, make_callback
        gc.collect()
        torch.cuda.empty_cache()
        return ms, times[len(times) // 2], e2e, stats

    def prefill_run(repeats: int = 5):
        engine = make_engine(1)
        generator = torch.Generator().manual_seed(2)
        prompt = torch.randint(0, config["vocab_size"], (PROMPT,), generator=generator).tolist()

        async def drive():
            try:
                for _ in range(repeats + 2):
                    await engine.generate(prompt, GenerationConfig(max_new_tokens=1, temperature=0.0))
                return engine.iteration_stats
            finally:
                await engine.close()

        asyncio.run(drive())
        times = sorted(a.elapsed_time(b) for a, b in engine._iteration_cuda_events["prefill"][2:])
        del engine, drive
        gc.collect()
        torch.cuda.empty_cache()
        return times[len(times) // 2]

    # The reference decorates its async ``_step`` with ``@torch.inference_mode()`` (``engine.py:244``); on a
    # coroutine function that only covers the creation of the coroutine, so its stock path runs with autograd on:
    # the in-place cache write (``kv_cache.py:265-266``) chains every step's graph to the cache tensor and the
    # activations of all earlier steps stay allocated (about 3 GB per 2,048-token step here).  ``value`` and ``e2e``
    # are that stock path; the same run under the driver's ``torch.inference_mode()`` is given beside it.  Batch 64
    # (65 prompt steps) runs out of 180 GB on the stock path and is measured under inference mode only.
    batch = args.batch
    stock = batch <= 16
    with ClockSampler() as clocks:
        ms, median_ms, e2e_value, stats = decode_run(batch, args.steps, args.warmup, inference_mode=not stock)
    guarded = None
    if stock:
        guarded_ms, _, guarded_e2e, _ = decode_run(batch, args.steps, args.warmup, inference_mode=True)
        guarded = {"value": round(batch / (guarded_ms / 1e3), 1), "ms_per_step": round(guarded_ms, 4), "e2e": round(guarded_e2e, 1)}
    kv_bytes = batch * (PROMPT + args.warmup + args.steps // 2 + batch) * kv_bytes_per_token
    achieved = (weight_bytes + kv_bytes) / (ms / 1e3) / 1e9
    prefill_ms = prefill_run()
    flops = prefill_flops(config, layers, PROMPT)
    points, notes = {}, {}
    for point_batch in (1, 64):
        try:
            point_ms, _, _, _ = decode_run(point_batch, max(args.steps // 2, 8), args.warmup, inference_mode=point_batch > 16)
            points[f"decode_b{point_batch}"] = round(point_batch / (point_ms / 1e3), 1)
            if point_batch > 16:
                notes[f"decode_b{point_batch}"] = "under the driver's torch.inference_mode()"
        except Exception as error:
            points[f"decode_b{point_batch}"] = None
            notes[f"decode_b{point_batch}"] = f"{type(error).__name__}: {str(error)[:160]}"
            torch.cuda.empty_cache()
    return {
        "metric": "decode tok/s at batch 8 (Qwen2.5-1.5B shape, 2,048-token prompts)",
        "value": round(batch / (ms / 1e3), 1), "unit": "tokens/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": round(ms, 4), "ms_per_step_median": round(median_ms, 4), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "fp16", "data": "synthetic (random weights, uniform random token ids)",
        "impl": "reference", "install": how, "attention_backend": backend,
        "config": bench_config(config, layers, batch),
        "prefill": {"value": round(PROMPT / (prefill_ms / 1e3), 1), "tokens": PROMPT, "ms": round(prefill_ms, 3),
                    "frac": round(flops / (prefill_ms / 1e3) / (peak["bf16_tflops"] * 1e12), 4)},
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": peak["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / peak["hbm_gbs"], 4), "peaks": peak["source"]},
        "points": points, "points_notes": notes,
        "autograd": "on (stock: the reference's inference_mode decorator sits on an async function and has no effect)" if stock
                    else "off (driver's torch.inference_mode())",
        "under_inference_mode": guarded,
        "e2e": {"value": round(e2e_value, 1), "unit": "tokens/s",
                "h2d_bytes_per_step": batch * (8 + 8 + 4 * 4), "d2h_bytes_per_step": batch * 8,
                "pipeline": "the reference's own loop: token ids, positions (int64) and four int32 metadata arrays from pinned "
                            "host memory every step, sampled ids back through .tolist()"},
        "iteration_stats": {key: (round(value, 3) if isinstance(value, float) else value) for key, value in stats.items()},
        "clocks": clocks.summary(),
    }


def timeline(args) -> int:
    """One decode step seen from the device: the tuning variant of the kernel library (built with
    ``-DLSE_TRACE``) lets block 0 of every kernel record when it started, when its wait for the kernels
    before returned and when it ended (nanoseconds of the global timer).  Prints the kernels of the first
    layers in order and the sums per kind of kernel."""
    import ctypes

    import torch

    os.environ["LSE_TRACE"] = "1"   # before the library is loaded
    from llm_serving_engine_b200.cache.manager import CacheManager
    from llm_serving_engine_b200.config.runtime_config import CacheConfig
    from llm_serving_engine_b200.engine.step import StepEntry, StepRunner
    from llm_serving_engine_b200.kernels import library
    from llm_serving_engine_b200.models import cache_requirements

    torch.cuda.set_device(0)
    lib = library.load()
    model, _ = build_model(args.layers or FULL_LAYERS, {"7b": QWEN25_7B_SIZES, "14b": QWEN25_14B_SIZES}.get(args.sizes))
    batch = args.batch
    context = model.spec.max_position_embeddings
    cache = CacheManager(cache_requirements(model.spec), CacheConfig(BLOCK, batch * (context // BLOCK)), model.dtype,
                         model.device, context, num_state_slots=batch)
    runner = StepRunner(model, cache, max(PROMPT, batch), batch, use_graphs=USE_GRAPHS)
    generator = torch.Generator().manual_seed(1)
    names = {1: "embedding", 2: "add+norm", 3: "rope+cache", 4: "silu", 5: "product", 6: "attention"}

    def read_all(reset: int):
        rows = []
        for reader in ("lse_timeline_elementwise", "lse_timeline_gemm", "lse_timeline_attention"):
            function = getattr(lib, reader)
            function.argtypes = [ctypes.c_void_p, ctypes.c_int]
            function.restype = ctypes.c_int
            buffer = (ctypes.c_ulonglong * (4096 * 8))()
            count = function(buffer, reset)
            rows += [tuple(int(buffer[i * 8 + k]) for k in range(4)) for i in range(count)]
        return sorted(rows, key=lambda row: row[1])

    ids = [f"r{index}" for index in range(batch)]
    with torch.inference_mode():
        for rid in ids:
            cache.create(rid)
            runner.run([StepEntry(rid, torch.randint(0, model.vocab_size, (PROMPT,), generator=generator).tolist(), [])])
        for _ in range(max(args.warmup, 3)):
            runner.run([StepEntry(rid, [5], [0]) for rid in ids])
        torch.cuda.synchronize()
        read_all(1)
        runner.run([StepEntry(rid, [5], [0]) for rid in ids])
        torch.cuda.synchronize()
    rows = read_all(1)
    origin = rows[0][1]
    print(f"decode step, batch {batch}, {len(rows)} kernels, {(max(row[3] for row in rows) - origin) / 1000:.1f} us "
          f"from the first kernel's start to the last kernel's end (block 0 of each; microseconds)")
    print(f"{'#':>3} {'kernel':10} {'started':>9} {'wait over':>10} {'ended':>9} {'after wait':>11} {'since the kernel before ended':>30}")
    before = origin
    for index, (kind, started, waited, ended) in enumerate(rows[:2 + 9 * args.timeline]):
        print(f"{index:3d} {names.get(kind, str(kind)):10} {(started - origin) / 1000:9.2f} {(waited - origin) / 1000:10.2f} "
              f"{(ended - origin) / 1000:9.2f} {(ended - waited) / 1000:11.2f} {(waited - before) / 1000:30.2f}")
        before = ended
    totals: dict[str, list] = {}
    before = origin
    for kind, started, waited, ended in rows:
        entry = totals.setdefault(names.get(kind, str(kind)), [0, 0.0, 0.0])
        entry[0] += 1
        entry[1] += (ended - waited) / 1000
        entry[2] += max(0.0, (waited - before) / 1000)
        before = ended
    for name, (count, active, gaps) in totals.items():
        print(f"{name:10} x{count:4d}: {active:8.1f} us after the wait in total, {active / count:6.2f} us each; "
              f"{gaps:8.1f} us between the kernel before and the wait's return")
    if args.timeline_json:
        # bytes a kind of kernel has to read in a step over the time its block 0 spends after its wait: a lower
        # bound of the kind's rate (other blocks end later; the first tiles were fetched before the wait)
        kv_bytes = batch * (PROMPT + max(args.warmup, 3) + 1) * cache.kv_bytes_per_token()
        moved = {"product": model.weight_bytes_per_step(), "attention": kv_bytes}
        table = {"step_us": round((max(row[3] for row in rows) - origin) / 1000, 1), "kernels_in_step": len(rows),
                 "how": "block 0 of every kernel stamps the global timer at its start, when its wait for the kernels "
                        "before returns and at its end (tuning variant of the library, one decode step from a CUDA graph)"}
        for name, (count, active, gaps) in totals.items():
            table[name] = {"launches": count, "us_after_wait": round(active, 1), "us_handover": round(gaps, 1)}
            if name in moved:
                table[name]["gb_per_s_after_wait"] = round(moved[name] / (active * 1e-6) / 1e9, 1)
        print(json.dumps(table))
    return 0


def main() -> int:
    parser = argparse.ArgumentParser()
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=64)
    parser.add_argument("--warmup", type=int, default=5)
    parser.add_argument("--impl", choices=("ours", "reference"), default="ours")
    parser.add_argument("--batch", type=int, default=8)
    parser.add_argument("--layers", type=int, default=0, help="fewer layers than the full model (0 = all)")
    parser.add_argument("--only", choices=("all", "decode", "prefill"), default="all",
                        help="run one part only (a small case for ncu; no bench line)")
    parser.add_argument("--no-graphs", action="store_true", help="decode launch by launch instead of from CUDA graphs")
    parser.add_argument("--sizes", choices=("1.5b", "7b", "14b"), default="1.5b",
                        help="layer sizes (7b, 14b: those of Qwen2.5-7B / 14B; only with --only, give --layers to fit the time)")
    parser.add_argument("--dtype", choices=("bfloat16", "float32"), default="bfloat16",
                        help="with --only: the true float32 path instead of the serving precision")
    parser.add_argument("--quick", action="store_true", help="the headline, its points and the end-to-end number only "
                                                             "(no other model sizes, no float32 point, no kernel table)")
    parser.add_argument("--design", choices=("givelix", "fororax", "tufevik", "sebudra"), default=None,
                        help="instead of the default workload: the named design at layer sizes of real models beside the "
                             "Qwen2 model of equal size (prefill and decode throughput, kernel times, rooflines)")
    parser.add_argument("--design-size", choices=tuple(sorted({name for sizes in DESIGN_SIZES.values() for name in sizes})),
                        default=None, help="with --design: one size only")
    parser.add_argument("--timeline-json", action="store_true", help="with --timeline: also one JSON line of sums per kind of kernel")
    parser.add_argument("--timeline", type=int, default=0, metavar="LAYERS",
                        help="print the device-side timeline of one decode step (the first LAYERS layers kernel by "
                             "kernel) from the tuning variant of the kernel library; no bench line")
    args = parser.parse_args()
    global USE_GRAPHS
    USE_GRAPHS = not args.no_graphs
    if args.sizes != "1.5b" and args.only == "all" and not args.timeline:
        print(f"--sizes {args.sizes} measures one part only: add --only decode or --only prefill")
        return 2
    if args.timeline:
        return timeline(args)
    if args.gpus != 1:
        print(f"bench.py measures a single-GPU engine; --gpus {args.gpus} is not supported")
        return 2
    if args.impl == "reference":
        args.warmup = max(args.warmup, 3)
        print(json.dumps(run_reference(args)))
        return 0
    if args.design:
        print(json.dumps(run_design(args)))
        return 0
    if args.only == "all":
        args.warmup = max(args.warmup, 3)
    print(json.dumps(run_ours(args)))
    return 0


if __name__ == "__main__":
    sys.exit(main())
