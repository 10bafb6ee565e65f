#!/usr/bin/env python3
"""Decode and prefill throughput of the engine at real Llama shapes with random weights, on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--batch 8] [--config tinyllama|llama2-7b|llama3-8b] [--layers L]
                    [--impl engine|reference]

One JSON line on standard output.  A "step" is one decode step of the whole batch.
  value      decoded tokens per second, timed on the device with CUDA events around K replays of
             the decode step (forward, sampling and advancing on the device, no host round trip);
  e2e        the same through the Python entry point (Engine.step): every step copies the input
             token ids from pinned host memory and reads the sampled ids back;
  prefill    one prompt of the configuration's prefill length through the step function, with the fraction of the tensor peak;
  roofline   bytes a decode step must read (every weight once + the cache of the live requests)
             divided by its time, against the measured copy bandwidth;
  points     decode tokens per second at batch 1 and 64 (with the vendor-library products each ran on).
The default configuration is TinyLlama 1.1B with all of its layers.  The larger shapes may run with fewer layers than the
checkpoints have (--layers); ``config`` then names both numbers, and every byte and flop count is of the layers that ran.
Between timed steps no cache flush is needed: a step reads gigabytes of weights, far more than
the 126 MB L2, so nothing survives from one step to the next.
``--impl reference`` runs the unmodified reference engine on the same metric (baseline/reference_arm.py).
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import tempfile
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

# The shapes the metric is quoted on (one table over sizes, as the reference's scripts/benchmark.py:32-36 has one over contexts):
# layer sizes of the checkpoint, the prompt length of the decode runs, the length of the timed prefill.
CONFIGS = {
    "tinyllama": dict(model="TinyLlama-1.1B shapes", prompt_tokens=1024, prefill_tokens=2048, default_layers=22,
                      shapes=dict(hidden_size=2048, intermediate_size=5632, num_hidden_layers=22, num_attention_heads=32, num_key_value_heads=4,
                                  max_position_embeddings=2048, vocab_size=32000, rms_norm_eps=1e-5, rope_theta=10000.0)),
    "llama2-7b": dict(model="Llama-2-7B shapes", prompt_tokens=1024, prefill_tokens=2048, default_layers=8,
                      shapes=dict(hidden_size=4096, intermediate_size=11008, num_hidden_layers=32, num_attention_heads=32, num_key_value_heads=32,
                                  max_position_embeddings=4096, vocab_size=32000, rms_norm_eps=1e-5, rope_theta=10000.0)),
    "llama3-8b": dict(model="Llama-3-8B shapes", prompt_tokens=7168, prefill_tokens=8192, default_layers=8,
                      shapes=dict(hidden_size=4096, intermediate_size=14336, num_hidden_layers=32, num_attention_heads=32, num_key_value_heads=8,
                                  max_position_embeddings=8192, vocab_size=128256, rms_norm_eps=1e-5, rope_theta=500000.0)),
}
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}


def peaks() -> tuple[dict, str]:
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        try:
            data = json.loads(path.read_text())
            flat = {}

            def walk(node):
                if isinstance(node, dict):
                    for key, value in node.items():
                        if isinstance(value, (int, float)) and key in ("hbm_gbs", "bf16_tflops", "bf16_tflops_sustained"):
                            flat.setdefault(key, float(value))
                        else:
                            walk(value)
                elif isinstance(node, list):
                    for value in node:
                        walk(value)

            walk(data)
            if "hbm_gbs" in flat and "bf16_tflops" in flat:
                return flat, "measured"
        except (OSError, ValueError):
            pass
    return dict(FALLBACK_PEAKS), "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons while a timed region runs (NVML reads only; nvidia-smi as a fallback)."""

    QUERY = "clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap"
    REASONS = {"hw_slowdown": 0x8, "hw_thermal_slowdown": 0x40, "sw_thermal_slowdown": 0x20, "sw_power_cap": 0x4}

    def __init__(self):
        self.clocks: list[int] = []
        self.max_clock = None
        self.reasons: set[str] = set()
        self._stop = threading.Event()
        self._thread = threading.Thread(target=self._run, daemon=True)
        self._nvml = None
        try:
            import pynvml

            pynvml.nvmlInit()
            self._nvml = pynvml
            self._handle = pynvml.nvmlDeviceGetHandleByIndex(0)
            self.max_clock = int(pynvml.nvmlDeviceGetMaxClockInfo(self._handle, pynvml.NVML_CLOCK_SM))
        except Exception:  # noqa: BLE001
            self._nvml = None

    def _sample_nvml(self) -> None:
        nv = self._nvml
        self.clocks.append(int(nv.nvmlDeviceGetClockInfo(self._handle, nv.NVML_CLOCK_SM)))
        try:
            mask = int(nv.nvmlDeviceGetCurrentClocksEventReasons(self._handle))
        except Exception:  # noqa: BLE001
            mask = int(nv.nvmlDeviceGetCurrentClocksThrottleReasons(self._handle))
        self.reasons |= {name for name, bit in self.REASONS.items() if mask & bit}

    def _sample_smi(self) -> None:
        out = subprocess.run(["nvidia-smi", "-i", "0", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits"],
                             capture_output=True, text=True, timeout=5).stdout.strip()
        if out:
            cells = [c.strip() for c in out.splitlines()[0].split(",")]
            if cells[0].isdigit():
                self.clocks.append(int(cells[0]))
            if cells[1].isdigit():
                self.max_clock = int(cells[1])
            self.reasons |= {name for name, flag in zip(self.REASONS, cells[2:6]) if flag.lower().startswith("active")}

    def _run(self):
        while not self._stop.is_set():
            try:
                self._sample_nvml() if self._nvml is not None else self._sample_smi()
            except Exception:  # noqa: BLE001
                return
            self._stop.wait(0.01 if self._nvml is not None else 0.2)

    def __enter__(self):
        self._thread.start()
        return self

    def __exit__(self, *exc):
        self._stop.set()
        self._thread.join(timeout=6)

    def summary(self) -> dict:
        clocks = sorted(self.clocks)
        return {"sm_mhz": clocks[len(clocks) // 2] if clocks else None, "sm_max_mhz": self.max_clock, "reasons": sorted(self.reasons), "samples": len(clocks)}


def model_folder(name: str, shapes: dict, layers: int) -> Path:
    """A random-weights model folder at the benchmark shapes (kept in the temporary folder between runs)."""
    from tinyllama_inference_engine_b200.weights import write_random_model

    suffix = "" if name == "tinyllama" else f"_{name}"
    folder = Path(tempfile.gettempdir()) / f"tlie_b200_bench_{os.getuid()}{suffix}_L{layers}"
    if not (folder / "model.safetensors").exists():
        staging = Path(tempfile.mkdtemp(prefix="tlie_b200_bench_", dir=tempfile.gettempdir()))
        write_random_model(staging, dict(shapes, num_hidden_layers=layers, architectures=["LlamaForCausalLM"], model_type="llama", bos_token_id=1, eos_token_id=2), seed=0)
        try:
            os.replace(staging, folder)
        except OSError:
            return staging if not (folder / "model.safetensors").exists() else folder
    return folder


def decode_bytes(shapes: dict, layers: int, batch: int, mean_context: float) -> float:
    """Bytes one decode step must read: every weight once, and the keys and values of the live requests."""
    h, i, v = shapes["hidden_size"], shapes["intermediate_size"], shapes["vocab_size"]
    d = h // shapes["num_attention_heads"]
    kv = shapes["num_key_value_heads"] * d
    per_layer = (h * (h + 2 * kv) + h * h + 2 * i * h + h * i) * 2 + 2 * h * 4
    weights = layers * per_layer + v * h * 2 + h * 4
    cache = batch * mean_context * layers * 2 * kv * 2
    return weights + cache


def prefill_flops(shapes: dict, layers: int, tokens: int) -> float:
    h, i, v = shapes["hidden_size"], shapes["intermediate_size"], shapes["vocab_size"]
    d = h // shapes["num_attention_heads"]
    kv = shapes["num_key_value_heads"] * d
    linear = 2.0 * tokens * (h * (h + 2 * kv) + h * h + 2 * i * h + h * i) * layers + 2.0 * v * h
    attention = 4.0 * shapes["num_attention_heads"] * d * tokens * (tokens + 1) / 2 * layers
    return linear + attention


def config_record(args, chosen: dict, layers: int, first_context: int, peak_kind: str) -> dict:
    """The sizes that were run, flat (nothing deeper survives in the record)."""
    shapes = chosen["shapes"]
    return {"model": chosen["model"], "layers": layers, "layers_of_model": shapes["num_hidden_layers"], "hidden": shapes["hidden_size"],
            "heads": shapes["num_attention_heads"], "kv_heads": shapes["num_key_value_heads"], "head_dim": shapes["hidden_size"] // shapes["num_attention_heads"],
            "intermediate": shapes["intermediate_size"], "vocab": shapes["vocab_size"], "global_batch": args.batch, "seq_len": shapes["max_position_embeddings"],
            "prompt_tokens": chosen["prompt_tokens"], "prefill_tokens": chosen["prefill_tokens"], "context_first_timed_step": first_context, "page_size": 64,
            "parallelism": "single GPU", "l2": "inputs larger than L2: each step streams gigabytes of weights", "peaks": peak_kind}


def metric_name(args, chosen: dict) -> str:
    if args.config == "tinyllama" and args.batch == 8:
        return "decode tokens/s at batch 8 (TinyLlama 1.1B shapes, 1,024-token prompts)"
    return f"decode tokens/s at batch {args.batch} ({chosen['model']}, {chosen['prompt_tokens']:,}-token prompts)"


def run_engine(args) -> dict:
    import numpy as np
    import torch

    from tinyllama_inference_engine_b200 import EngineConfig
    from tinyllama_inference_engine_b200.engine.api import Engine
    from tinyllama_inference_engine_b200.engine.batch import StepEntry
    from tinyllama_inference_engine_b200.engine.decode_session import DecodeSession
    from tinyllama_inference_engine_b200.engine.request import SamplingParams

    chosen = CONFIGS[args.config]
    shapes, prompt_tokens, prefill_tokens = chosen["shapes"], chosen["prompt_tokens"], chosen["prefill_tokens"]
    layers, steps, warmup = args.layers or chosen["default_layers"], args.steps, args.warmup
    folder = model_folder(args.config, shapes, layers)
    rng = np.random.default_rng(0)
    vocab = shapes["vocab_size"]
    generated = warmup + steps + 8   # requests whose prompts ran in different steps are a few tokens apart: none finishes inside the timed steps
    if prompt_tokens + generated > shapes["max_position_embeddings"]:
        raise SystemExit(f"warmup + steps must stay within the {shapes['max_position_embeddings']:,}-token context after a {prompt_tokens:,}-token prompt")

    def prompts(count, length):
        return [[int(t) for t in rng.integers(0, vocab, size=length)] for _ in range(count)]

    def event_ms(fn) -> float:
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        start.record()
        fn()
        end.record()
        torch.cuda.synchronize()
        return start.elapsed_time(end)

    sections = set(args.sections.split(","))
    largest = max(64 if "points" in sections else 1, args.batch)
    cache_tokens = largest * (prompt_tokens + 64 * (-(-generated // 64)) + 64)
    # Requests of mixed length for the scheduler (prompts uniform between 64 tokens and the context, cut into
    # portions under the token budget and interleaved with the other requests' decode steps); all of them fit the cache at once.
    mixed_count, mixed_out = 32, 64
    mixed_lengths = [int(n) for n in rng.integers(64, min(4096, shapes["max_position_embeddings"] - mixed_out - 1) + 1, size=mixed_count)]
    if "mixed" in sections:
        largest = max(largest, mixed_count)
        cache_tokens = max(cache_tokens, sum(64 * (-(-(n + mixed_out) // 64)) + 64 for n in mixed_lengths))
    config = EngineConfig(dtype="bfloat16", page_size=64, max_cache_tokens=cache_tokens, max_requests=largest, max_batch_tokens=max(prefill_tokens, prompt_tokens))
    engine = Engine(folder, config)
    runner = engine.runner

    library_per_step: dict[int, int] = {}

    def device_decode(batch: int) -> tuple[float, float, int, dict]:
        """Tokens per second of K decode steps kept on the device; also ms per step, kernels per step, clocks."""
        ids = [f"d{batch}-{i}" for i in range(batch)]
        for rid, prompt in zip(ids, prompts(batch, prompt_tokens)):
            runner.step([StepEntry(rid, prompt, [])])
        session = DecodeSession(runner, batch, publish=False)   # these steps stay on the device: nothing goes to host memory
        session.load(ids, [int(t) for t in rng.integers(0, vocab, size=batch)], [SamplingParams()] * batch, [0] * batch)
        for _ in range(max(warmup, 3)):
            session.step()
        with ClockSampler() as clocks:
            ms = event_ms(lambda: [session.step() for _ in range(steps)])
        for rid in ids:
            runner.finish(rid)
        library_per_step[batch] = session.library_calls_per_step
        return batch * steps / (ms / 1e3), ms / steps, session.kernels_per_step, clocks.summary()

    value, ms_per_step, kernels_per_step, clocks = device_decode(args.batch) if "decode" in sections else (0.0, 1.0, 0, {})
    first_context = prompt_tokens + max(warmup, 3)
    mean_context = first_context + (steps + 1) / 2.0
    step_bytes = decode_bytes(shapes, layers, args.batch, mean_context)
    peak, peak_kind = peaks()
    achieved = step_bytes / (ms_per_step / 1e3) / 1e9

    # the same through the Python entry point: host token ids in, sampled ids out, every step
    e2e = None
    if "e2e" in sections:
        ids = [engine.add_request(p, SamplingParams(max_tokens=generated)) for p in prompts(args.batch, prompt_tokens)]
        while any(not engine.requests[i].generated for i in ids):
            engine.step()
        for _ in range(max(warmup, 3)):
            engine.step()
        torch.cuda.synchronize()
        started = time.perf_counter()
        for _ in range(steps):
            engine.step()
        torch.cuda.synchronize()
        e2e_seconds = time.perf_counter() - started
        for i in ids:
            engine.cancel(i)
        e2e = {"value": args.batch * steps / e2e_seconds, "unit": "tokens/s", "h2d_bytes_per_step": args.batch * 4, "d2h_bytes_per_step": (args.batch + 2) * 4}   # ids in; ids, the device error word and the step number out

    # prefill of one prompt
    prefill = None
    if "prefill" in sections:
        prefill_ms = []
        for index, prompt in enumerate(prompts(3 + args.prefill_samples, prefill_tokens)):
            rid = f"p{index}"
            prefill_ms.append(event_ms(lambda: runner.step([StepEntry(rid, prompt, [prefill_tokens - 1])])))
            runner.finish(rid)
        timed = sorted(prefill_ms[3:])
        best = timed[len(timed) // 2]
        flops = prefill_flops(shapes, layers, prefill_tokens)
        prefill = {"value": prefill_tokens / (best / 1e3), "tokens": prefill_tokens, "ms": best,
                   "frac": flops / (best / 1e3) / (peak["bf16_tflops"] * 1e12), "tflops": flops / (best / 1e3) / 1e12}

    points = {}
    if "points" in sections:
        for batch in (1, 64):
            if batch == args.batch:
                points[f"decode_b{batch}"] = value
                points[f"decode_b{batch}_hbm_frac"] = achieved / peak["hbm_gbs"]
            else:
                tokens_per_s, ms, _, _ = device_decode(batch)
                points[f"decode_b{batch}"] = tokens_per_s
                points[f"decode_b{batch}_hbm_frac"] = decode_bytes(shapes, layers, batch, mean_context) / (ms / 1e3) / 1e9 / peak["hbm_gbs"]
            points[f"decode_b{batch}_library_gemms_per_step"] = library_per_step.get(batch, 0)

    if "mixed" in sections:
        count, out_tokens, lengths = mixed_count, mixed_out, mixed_lengths
        requests = [[int(t) for t in rng.integers(0, vocab, size=n)] for n in lengths]
        for run in range(4):   # the first runs build kernels and meet every step shape and batch size (graphs are captured on the third use)
            steps_before = runner.steps
            torch.cuda.synchronize()
            started = time.perf_counter()
            results = engine.generate(requests, SamplingParams(max_tokens=out_tokens))
            torch.cuda.synchronize()
            seconds = time.perf_counter() - started
        points["mixed_requests"] = count
        points["mixed_prompt_tokens"] = sum(lengths)
        points["mixed_generated_tokens"] = sum(len(r.generated_tokens) for r in results)
        points["mixed_steps"] = runner.steps - steps_before
        points["mixed_preemptions"] = sum(r.preemptions for r in results)
        points["mixed_tokens_per_s"] = (sum(lengths) + points["mixed_generated_tokens"]) / seconds
        points["mixed_generated_per_s"] = points["mixed_generated_tokens"] / seconds

    return {
        "metric": metric_name(args, chosen),
        "value": value, "unit": "tokens/s", "n_gpus": 1, "steps": steps, "warmup": max(warmup, 3), "ms_per_step": ms_per_step,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic (random weights N(0, 0.02), uniform random token ids)",
        "impl": "engine",
        "config": config_record(args, chosen, layers, first_context, peak_kind),
        "e2e": e2e,
        "gpu_launches": kernels_per_step * steps,
        "library_gemms_per_step": library_per_step.get(args.batch, 0),
        "prefill": prefill,
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak["hbm_gbs"], "unit": "GB/s", "frac": achieved / peak["hbm_gbs"], "bytes_per_step": step_bytes},
        "points": points,
        "clocks": clocks,
    }


# --- another design beside the closest existing one ---------------------------------------------------------------------------
# `--designs`: Marutar (minGRU layers and attention with mixed heads, a sliding window and an output gate) at sizes that resemble
# real models' layers, beside the Llama decoder at equal width, heads, feed-forward and layer count: prompt and decode throughput
# through the same engine, and the design's own kernels alone beside the like kernels of the Llama path, each against its roofline.
DESIGN_SIZES = {
    "w2048": dict(width=2048, recurrent=2048, heads=32, kv_heads=4, dim=64, vdim=64, window=1024, ff=5632, vocab=32000, positions=4096, layers=8,
                  pattern=("mingru", "mingru", "attention", "mingru")),
    "w4096": dict(width=4096, recurrent=4096, heads=32, kv_heads=8, dim=128, vdim=128, window=2048, ff=14336, vocab=32000, positions=4096, layers=4,
                  pattern=("mingru", "attention")),
}


def design_configs(size: dict) -> tuple[dict, dict]:
    """config.json of the Marutar model and of the Llama model of equal width, heads, feed-forward and layer count."""
    layers = []
    for index in range(size["layers"]):
        kind = size["pattern"][index % len(size["pattern"])]
        if kind == "mingru":
            layers.append({"type": "mingru", "mixer": {"width": size["recurrent"]}, "mlp": {"kind": "dense", "ff": size["ff"]}})
        else:
            layers.append({"type": "attention", "mixer": {"heads": size["heads"], "kv_heads": size["kv_heads"], "dim": size["dim"], "vdim": size["vdim"],
                                                          "scale": size["dim"] ** -0.5, "mask": {"size": size["window"]}}, "mlp": {"kind": "dense", "ff": size["ff"]}})
    marutar = {"architecture": "Marutar", "vocab": size["vocab"], "width": size["width"], "max_positions": size["positions"], "norm": {"eps": 1e-5}, "layers": layers}
    llama = dict(architectures=["LlamaForCausalLM"], model_type="llama", hidden_size=size["width"], intermediate_size=size["ff"], num_hidden_layers=size["layers"],
                 num_attention_heads=size["heads"], num_key_value_heads=size["kv_heads"], head_dim=size["dim"], max_position_embeddings=size["positions"],
                 vocab_size=size["vocab"], rms_norm_eps=1e-5, rope_theta=10000.0, bos_token_id=1, eos_token_id=2)
    return marutar, llama


# `--designs zirutar`: Zirutar (the gated delta rule, attention with normalised keys under a window that keeps the first tokens, latent
# attention with a sink; clamped gated feed-forwards; a gated slice of a second token table per layer) beside Marutar, the closest of
# the engine's designs (a recurrence per request and windowed, gated attention over pages), at equal width, feed-forward width, layer
# count, vocabulary and attention heads.
ZIRUTAR_SIZES = {
    "w2048": dict(delta_heads=16, delta_dim=128, delta_vdim=128, taps=4, low_rank=64, latent_heads=16, plain=128, rot=64, latent_vdim=128, rank=512, keep=4, side=256,
                  limit=7.0, pattern=("channel_delta", "channel_delta", "attention", "latent_attention")),
    "w4096": dict(delta_heads=32, delta_dim=128, delta_vdim=128, taps=4, low_rank=128, latent_heads=16, plain=128, rot=64, latent_vdim=128, rank=512, keep=4, side=256,
                  limit=7.0, pattern=("channel_delta", "attention", "latent_attention", "attention")),
}


def zirutar_config(size: dict, extra: dict) -> dict:
    layers = []
    for index in range(size["layers"]):
        kind = extra["pattern"][index % len(extra["pattern"])]
        if kind == "channel_delta":
            mixer = {"heads": extra["delta_heads"], "kv_heads": extra["delta_heads"], "dim": extra["delta_dim"], "vdim": extra["delta_vdim"], "conv": extra["taps"],
                     "decay_rank": extra["low_rank"], "gate_rank": extra["low_rank"]}
        elif kind == "attention":
            mixer = {"heads": size["heads"], "kv_heads": size["kv_heads"], "dim": size["dim"], "vdim": size["dim"], "scale": size["dim"] ** -0.5,
                     "mask": {"size": size["window"], "keep_first": extra["keep"]}}
        else:
            mixer = {"heads": extra["latent_heads"], "dim": extra["plain"], "rot_dim": extra["rot"], "vdim": extra["latent_vdim"], "kv_rank": extra["rank"],
                     "scale": (extra["plain"] + extra["rot"]) ** -0.5, "rot": {"base": 10000.0, "dims": extra["rot"]}}
        layers.append({"type": kind, "mixer": mixer, "mlp": {"kind": "dense", "ff": size["ff"], "limit": extra["limit"]}})
    return {"architecture": "Zirutar", "vocab": size["vocab"], "width": size["width"], "norm": {"eps": 1e-5}, "embedding": {"scale": size["width"] ** 0.5},
            "logit_scale": 1.0, "token_side": {"dim": extra["side"]}, "layers": layers}


# `--designs redasun`: Redasun (differential attention with normalised, partly rotated queries and keys; layer norms before and after
# every sublayer; gated feed-forwards with gelu, every second layer a mixture of experts with a shared expert) beside the Llama decoder, the
# closest of the engine's designs (rotary grouped-query attention and a gated feed-forward), at equal width, layer count and vocabulary,
# as many query and key vectors per token (two per head here) and as wide a feed-forward per token (the chosen experts' widths add up to it).
REDASUN_SIZES = {
    "w2048": dict(heads=16, kv_heads=2, dim=64, vdim=128, rot=32, experts=32, top=4, groups=(8, 4), expert_ff=1408, shared_ff=1408),
    "w4096": dict(heads=16, kv_heads=4, dim=128, vdim=128, rot=64, experts=32, top=4, groups=(8, 4), expert_ff=3584, shared_ff=3584),
}


def redasun_config(size: dict, extra: dict) -> dict:
    layers = []
    for index in range(size["layers"]):
        mixer = {"heads": extra["heads"], "kv_heads": extra["kv_heads"], "dim": extra["dim"], "vdim": extra["vdim"], "scale": extra["dim"] ** -0.5, "diff": 0.5,
                 "rot": {"base": 10000.0, "dims": extra["rot"]}}
        if index % 2 == 0:
            mlp = {"kind": "dense", "ff": size["ff"]}
        else:
            mlp = {"kind": "moe", "expert": {"ff": extra["expert_ff"]}, "shared": {"ff": extra["shared_ff"]},
                   "router": {"experts": extra["experts"], "top": extra["top"], "scale": 2.0, "groups": {"count": extra["groups"][0], "keep": extra["groups"][1]}}}
        layers.append({"type": "attention", "mixer": mixer, "mlp": mlp})
    return {"architecture": "Redasun", "vocab": size["vocab"], "width": size["width"], "norm": {"eps": 1e-5}, "embedding": {"scale": size["width"] ** 0.5}, "layers": layers}


# `--designs kilurax`: Kilurax (softmax attention with biased projections and a partial rotation side by side with a state-space layer; a
# linear-attention layer whose forget gate also writes; the gated delta rule with one decay per head; grouped RMS norms before and after every
# sublayer, a short convolution in front of each; a mixture of experts that read their token times its score, beside a shared expert, in every
# layer; an embedding that also reads the token before) beside Redasun, the closest of the engine's designs (norms before and after every
# sublayer, attention over pages, a mixture of experts beside a shared one), at equal width, layer count and vocabulary and as wide experts.
KILURAX_SIZES = {
    "w2048": dict(left=dict(heads=16, kv_heads=4, dim=128, vdim=128, rot=64), right=dict(heads=32, vdim=64, state=128, groups=1, conv=4, norm_groups=1),
                  hgrn2=dict(heads=16, dim=128, vdim=128), delta=dict(heads=16, kv_heads=16, dim=128, vdim=128, conv=4), experts=32, top=4, expert_ff=1408, shared_ff=1408,
                  norm_groups=4, taps=3, pattern=("parallel", "hgrn2", "delta", "hgrn2")),
    "w4096": dict(left=dict(heads=32, kv_heads=8, dim=128, vdim=128, rot=64), right=dict(heads=64, vdim=64, state=128, groups=1, conv=4, norm_groups=1),
                  hgrn2=dict(heads=32, dim=128, vdim=128), delta=dict(heads=32, kv_heads=32, dim=128, vdim=128, conv=4), experts=32, top=4, expert_ff=3584, shared_ff=3584,
                  norm_groups=4, taps=3, pattern=("parallel", "delta", "hgrn2", "parallel")),
}


def kilurax_config(size: dict, extra: dict) -> dict:
    layers = []
    for index in range(size["layers"]):
        kind = extra["pattern"][index % len(extra["pattern"])]
        if kind == "parallel":
            left, right = extra["left"], extra["right"]
            mixer = {"left": {"heads": left["heads"], "kv_heads": left["kv_heads"], "dim": left["dim"], "vdim": left["vdim"], "scale": left["dim"] ** -0.5,
                              "rot": {"base": 10000.0, "dims": left["rot"]}}, "right": dict(right), "left_scale": 0.7, "right_scale": 0.7}
        else:
            mixer = dict(extra[kind])
        mlp = {"kind": "moe", "expert": {"ff": extra["expert_ff"]}, "shared": {"ff": extra["shared_ff"]}, "router": {"experts": extra["experts"], "top": extra["top"]}}
        layers.append({"type": kind, "mixer": mixer, "mlp": mlp})
    return {"architecture": "Kilurax", "vocab": size["vocab"], "width": size["width"], "norm": {"eps": 1e-5, "groups": extra["norm_groups"]}, "residual_mult": 0.5,
            "embedding": {"scale": size["width"] ** 0.5, "bigram": {"buckets": 65521, "mul_prev": 31, "mul_cur": 7}}, "canon": {"taps": extra["taps"]}, "layers": layers}


def run_designs(args) -> dict:
    import numpy as np
    import torch

    from tinyllama_inference_engine_b200 import EngineConfig, ops
    from tinyllama_inference_engine_b200.engine.batch import StepEntry, pack_step
    from tinyllama_inference_engine_b200.engine.decode_session import DecodeSession
    from tinyllama_inference_engine_b200.engine.request import SamplingParams
    from tinyllama_inference_engine_b200.engine.runner import ModelRunner
    from tinyllama_inference_engine_b200.ops import fast
    from tinyllama_inference_engine_b200.parts.base import CacheNeed, LayerCache
    from tinyllama_inference_engine_b200.weights import write_random_model

    peak, peak_kind = peaks()
    device = torch.device("cuda:0")
    rng = np.random.default_rng(0)
    flush = torch.empty(1 << 30, dtype=torch.uint8, device=device)   # larger than L2, written before every timed launch; long enough a write that the host has the launch queued when it ends
    prompt_tokens, context, batch, steps = 2048, 1024, args.batch, min(args.steps, 64)

    def timed(fn, repeats=7) -> float:
        """Median device time (ms) of ``fn`` alone, L2 flushed before every launch."""
        times = []
        for index in range(3 + repeats):
            flush.zero_()
            start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record()
            fn()
            end.record()
            torch.cuda.synchronize()
            if index >= 3:
                times.append(start.elapsed_time(end))
        return sorted(times)[len(times) // 2]

    def model_numbers(folder) -> dict:
        runner = ModelRunner(folder, EngineConfig(dtype="bfloat16", page_size=64, max_cache_tokens=batch * (context + 256) + prompt_tokens + 64, max_requests=batch + 1,
                                                  max_batch_tokens=prompt_tokens))
        vocab = runner.spec.vocab_size
        prompt_ms = []
        for index in range(8):   # the shape repeats: from its second use on the step is a replayed graph, for both designs alike
            tokens = [int(t) for t in rng.integers(0, vocab, size=prompt_tokens)]
            flush.zero_()
            start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record()
            runner.step([StepEntry(f"p{index}", tokens, [prompt_tokens - 1])])
            end.record()
            torch.cuda.synchronize()
            prompt_ms.append(start.elapsed_time(end))
            runner.finish(f"p{index}")
        prefill = sorted(prompt_ms[3:])[len(prompt_ms[3:]) // 2]
        ids = [f"d{i}" for i in range(batch)]
        for rid in ids:
            runner.step([StepEntry(rid, [int(t) for t in rng.integers(0, vocab, size=context)], [])])
        session = DecodeSession(runner, batch, publish=False)
        session.load(ids, [int(t) for t in rng.integers(0, vocab, size=batch)], [SamplingParams()] * batch, [0] * batch)
        for _ in range(4):
            session.step()
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        start.record()
        for _ in range(steps):
            session.step()
        end.record()
        torch.cuda.synchronize()
        decode_ms = start.elapsed_time(end) / steps
        weights = sum(t.numel() * t.element_size() for part in [runner.model.embedding, *runner.model.blocks, runner.model.head] for t in _tensors_of(part))
        out = {"prefill_ms": prefill, "prefill_tokens_per_s": prompt_tokens / (prefill / 1e3), "decode_ms_per_step": decode_ms, "decode_tokens_per_s": batch / (decode_ms / 1e3),
               "weight_bytes": weights, "decode_hbm_frac": weights / (decode_ms / 1e3) / 1e9 / peak["hbm_gbs"], "kernels_per_decode_step": session.kernels_per_step,
               "library_gemms_per_decode_step": session.library_calls_per_step}
        del session, runner
        torch.cuda.empty_cache()
        return out

    def _tensors_of(part, seen=None):
        seen = set() if seen is None else seen
        for value in vars(part).values():
            if isinstance(value, torch.Tensor) and value.data_ptr() not in seen:
                seen.add(value.data_ptr())
                yield value
            elif hasattr(value, "runtime") and hasattr(value, "spec"):
                yield from _tensors_of(value, seen)

    def kernel_numbers(size: dict) -> dict:
        """The design's own kernels alone, and the Llama path's attention kernels at the same heads, widths and window."""
        H, G, D, VD, W, R = size["heads"], size["kv_heads"], size["dim"], size["vdim"], size["window"], size["recurrent"]
        page, bf16 = 64, torch.bfloat16
        out = {}
        pages_needed = -(-(context + 1) // page) * batch + -(-prompt_tokens // page)
        pages = torch.randn(pages_needed, 2, G, page, D, dtype=torch.float32, device=device).to(bf16)
        slopes = torch.tensor([2.0 ** (-8.0 * (h + 1) / H) for h in range(H)], dtype=torch.float32, device=device)
        mix = (torch.randn(H, H, device=device) * H ** -0.5).contiguous()
        folded = fast.folded_slopes(slopes, mix)

        def context_for(lens, firsts):
            table_width = size["positions"] // page
            rows, at = [], 0
            for n, f in zip(lens, firsts):
                count = -(-(f + n) // page)
                rows.append(list(range(at, at + count)) + [-1] * (table_width - count))
                at += count
            entries = [StepEntry(i, [0] * n, []) for i, n in enumerate(lens)]
            return pack_step(entries, list(firsts), list(range(len(lens))), [rows], device)

        for name, lens, firsts in (("prefill", [prompt_tokens], [0]), ("decode", [1] * batch, [context] * batch)):
            ctx = context_for(lens, firsts)
            tokens = sum(lens)
            cache = LayerCache(CacheNeed("pages"), True, pages, ctx.block_tables[0], page)
            visible = sum(min(f + i + 1, W) for n, f in zip(lens, firsts) for i in range(n))
            rows = torch.randn(tokens, H * D + G * D + G * VD + H * VD, device=device).to(bf16)
            mixed = torch.empty(tokens, H * VD, dtype=bf16, device=device)
            ms = timed(lambda: ops.mixed_heads_attention(rows, H * D + G * D + G * VD, ctx.positions, ctx.token_seq, cache, slopes, mix, mixed, H, G, D, VD, W, D ** -0.5,
                                                         batch=ctx, folded_slopes=folded))
            qkv = torch.randn(tokens, (H + 2 * G) * D, device=device).to(bf16)
            plain = torch.empty(tokens, H * D, dtype=bf16, device=device)
            like_ms = timed(lambda: ops.paged_attention(qkv, pages, ctx.positions, ctx.token_seq, ctx.block_tables[0], plain, H, G, D, page, W, D ** -0.5, batch=ctx))
            if name == "prefill":
                flops, like_flops = visible * H * (2.0 * (D + VD) + 2.0 * H), visible * H * 4.0 * D
                out["attention_prefill"] = {"ms": ms, "tflops": flops / ms / 1e9, "frac": flops / (ms / 1e3) / (peak["bf16_tflops"] * 1e12),
                                            "like_ms": like_ms, "like_tflops": like_flops / like_ms / 1e9, "like_frac": like_flops / (like_ms / 1e3) / (peak["bf16_tflops"] * 1e12)}
            else:
                moved = visible * G * (D + VD) * 2.0
                out["attention_decode"] = {"ms": ms, "gbs": moved / ms / 1e6, "frac": moved / (ms / 1e3) / 1e9 / peak["hbm_gbs"],
                                           "like_ms": like_ms, "like_gbs": moved / like_ms / 1e6, "like_frac": moved / (like_ms / 1e3) / 1e9 / peak["hbm_gbs"]}
            zxg = torch.randn(tokens, 3 * R, device=device).to(bf16)
            gated = torch.empty(tokens, R, dtype=bf16, device=device)
            state = torch.zeros(batch + 1, R, device=device)
            bias = torch.zeros(R, device=device)
            scan_ms = timed(lambda: ops.mingru_scan(zxg, bias, bias, state, ctx.seq_starts, ctx.state_slots, gated, max(lens)))
            moved = tokens * 4.0 * R * 2 + (len(lens) * R * 8 if name == "decode" else 0)
            out[f"mingru_scan_{name}"] = {"ms": scan_ms, "gbs": moved / scan_ms / 1e6, "frac": moved / (scan_ms / 1e3) / 1e9 / peak["hbm_gbs"]}
        return out

    def zirutar_kernel_numbers(size: dict, extra: dict) -> dict:
        """Zirutar's own kernels alone against their rooflines, beside Marutar's like kernels (its attention at the same heads, widths and
        window; its scan over as many channels as the delta rule has value channels)."""
        H, G, D, W = size["heads"], size["kv_heads"], size["dim"], size["window"]
        DH, DD, DV = extra["delta_heads"], extra["delta_dim"], extra["delta_vdim"]
        LH, rank, rot = extra["latent_heads"], extra["rank"], extra["rot"]
        page, bf16 = 64, torch.bfloat16
        out = {}
        pages_needed = -(-(context + 1) // page) * batch + -(-prompt_tokens // page)
        pages = torch.randn(pages_needed, 2, G, page, D, dtype=torch.float32, device=device).to(bf16)
        latent_pages = torch.randn(pages_needed, 1, 1, page, rank + rot, dtype=torch.float32, device=device).to(bf16)
        slopes = torch.tensor([2.0 ** (-8.0 * (h + 1) / H) for h in range(H)], dtype=torch.float32, device=device)
        mix = (torch.randn(H, H, device=device) * H ** -0.5).contiguous()
        folded = fast.folded_slopes(slopes, mix)
        sinks = torch.zeros(LH, device=device)

        def context_for(lens, firsts):
            table_width = size["positions"] // page
            rows, at = [], 0
            for n, f in zip(lens, firsts):
                count = -(-(f + n) // page)
                rows.append(list(range(at, at + count)) + [-1] * (table_width - count))
                at += count
            entries = [StepEntry(i, [0] * n, []) for i, n in enumerate(lens)]
            return pack_step(entries, list(firsts), list(range(len(lens))), [rows], device)

        for name, lens, firsts in (("prefill", [prompt_tokens], [0]), ("decode", [1] * batch, [context] * batch)):
            ctx = context_for(lens, firsts)
            tokens = sum(lens)
            cache = LayerCache(CacheNeed("pages"), True, pages, ctx.block_tables[0], page)
            latent_cache = LayerCache(CacheNeed("pages"), True, latent_pages, ctx.block_tables[0], page)
            windowed = sum(min(f + i + 1, W) for n, f in zip(lens, firsts) for i in range(n))
            causal = sum(f + i + 1 for n, f in zip(lens, firsts) for i in range(n))
            width = -(-(H * D + G * D + H) // 8) * 8
            rows = torch.randn(tokens, width, device=device).to(bf16)
            mixed = torch.empty(tokens, H * D, dtype=bf16, device=device)
            ms = timed(lambda: ops.mixed_heads_attention(rows, H * D + G * D, ctx.positions, ctx.token_seq, cache, None, None, mixed, H, G, D, D, W, D ** -0.5, batch=ctx,
                                                         keep_first=extra["keep"], gate_per_head=True))
            like_rows = torch.randn(tokens, H * D + 2 * G * D + H * D, device=device).to(bf16)
            like_ms = timed(lambda: ops.mixed_heads_attention(like_rows, H * D + 2 * G * D, ctx.positions, ctx.token_seq, cache, slopes, mix, mixed, H, G, D, D, W, D ** -0.5,
                                                              batch=ctx, folded_slopes=folded))
            queries = torch.randn(tokens, LH * (rank + rot), device=device).to(bf16)
            summed = torch.empty(tokens, LH * rank, dtype=bf16, device=device)
            latent_ms = timed(lambda: ops.mixed_heads_attention(queries, -1, ctx.positions, ctx.token_seq, latent_cache, None, None, summed, LH, 1, rank + rot, rank, 0,
                                                                (extra["plain"] + rot) ** -0.5, batch=ctx, sinks=sinks, values_in_keys=True))
            if name == "prefill":
                flops, like_flops = windowed * H * 4.0 * D, windowed * H * (4.0 * D + 2.0 * H)
                latent_flops = causal * LH * 2.0 * (2 * rank + rot)
                out["attention_prefill"] = {"ms": ms, "tflops": flops / ms / 1e9, "frac": flops / (ms / 1e3) / (peak["bf16_tflops"] * 1e12),
                                            "like_ms": like_ms, "like_tflops": like_flops / like_ms / 1e9, "like_frac": like_flops / (like_ms / 1e3) / (peak["bf16_tflops"] * 1e12)}
                out["latent_attention_prefill"] = {"ms": latent_ms, "tflops": latent_flops / latent_ms / 1e9, "frac": latent_flops / (latent_ms / 1e3) / (peak["bf16_tflops"] * 1e12)}
            else:
                moved = windowed * G * 2 * D * 2.0
                latent_moved = causal * (rank + rot) * 2.0
                out["attention_decode"] = {"ms": ms, "gbs": moved / ms / 1e6, "frac": moved / (ms / 1e3) / 1e9 / peak["hbm_gbs"],
                                           "like_ms": like_ms, "like_gbs": moved / like_ms / 1e6, "like_frac": moved / (like_ms / 1e3) / 1e9 / peak["hbm_gbs"]}
                out["latent_attention_decode"] = {"ms": latent_ms, "gbs": latent_moved / latent_ms / 1e6, "frac": latent_moved / (latent_ms / 1e3) / 1e9 / peak["hbm_gbs"]}
            # the delta rule's recurrence, and Marutar's scan over as many channels as the rule has value channels
            channels = 2 * DH * DD + DH * DV
            prep = torch.rand(tokens, channels + DH + DH * DD, device=device)
            words, _ = ops.delta_state_words(DH, DD, DV, channels, extra["taps"])
            state = torch.zeros(batch + 1, words, device=device)
            read = torch.empty(tokens, DH * DV, device=device)
            rule_ms = timed(lambda: ops.delta_rule(prep, state, ctx, read, DH, DH, DD, DV))
            rule_flops = tokens * DH * DD * DV * 7.0
            rule_moved = tokens * 4.0 * (prep.shape[1] + DH * DV) + len(lens) * DH * DD * DV * 8.0
            R = DH * DV
            zxg = torch.randn(tokens, 3 * R, device=device).to(bf16)
            gated = torch.empty(tokens, R, dtype=bf16, device=device)
            scan_state = torch.zeros(batch + 1, R, device=device)
            bias = torch.zeros(R, device=device)
            scan_ms = timed(lambda: ops.mingru_scan(zxg, bias, bias, scan_state, ctx.seq_starts, ctx.state_slots, gated, max(lens)))
            scan_moved = tokens * 4.0 * R * 2 + (len(lens) * R * 8 if name == "decode" else 0)
            out[f"delta_rule_{name}"] = {"ms": rule_ms, "gbs": rule_moved / rule_ms / 1e6, "frac": rule_moved / (rule_ms / 1e3) / 1e9 / peak["hbm_gbs"],
                                         "fp32_tflops": rule_flops / rule_ms / 1e9, "like_ms": scan_ms, "like_gbs": scan_moved / scan_ms / 1e6,
                                         "like_frac": scan_moved / (scan_ms / 1e3) / 1e9 / peak["hbm_gbs"]}
        return out

    def redasun_kernel_numbers(size: dict, extra: dict) -> dict:
        """Redasun's own kernels alone against their rooflines, beside the Llama path's like kernels: its attention at as many query and key
        vectors of the same width, its gated feed-forward's products at the width the chosen experts add up to."""
        H, G, D, VD = extra["heads"], extra["kv_heads"], extra["dim"], extra["vdim"]
        LH, LG = 2 * H, 2 * G                         # the Llama path's heads: as many query and key vectors of width D
        E, top, F, W = extra["experts"], extra["top"], extra["expert_ff"], size["width"]
        page, bf16 = 64, torch.bfloat16
        out = {}
        pages_needed = -(-(context + 1) // page) * batch + -(-prompt_tokens // page)
        planes = (torch.randn(pages_needed, 2 * G, page, D, device=device).to(bf16), torch.randn(pages_needed, G, page, VD, device=device).to(bf16))
        like_pages = torch.randn(pages_needed, 2, LG, page, D, device=device).to(bf16)
        inv_freq = torch.tensor([10000.0 ** (-2.0 * i / extra["rot"]) for i in range(extra["rot"] // 2)], dtype=torch.float32, device=device)
        ones = torch.ones(D, device=device)
        gate_up = (torch.randn(E, 2 * F, W, device=device) * W ** -0.5).to(bf16)
        down = (torch.randn(E, W, F, device=device) * F ** -0.5).to(bf16)
        router = torch.randn(E, W, device=device) * W ** -0.5
        like_gate_up = (torch.randn(2 * top * F, W, device=device) * W ** -0.5).to(bf16)
        like_down = (torch.randn(W, top * F, device=device) * F ** -0.5).to(bf16)

        def context_for(lens, firsts):
            table_width = size["positions"] // page
            rows, at = [], 0
            for n, f in zip(lens, firsts):
                count = -(-(f + n) // page)
                rows.append(list(range(at, at + count)) + [-1] * (table_width - count))
                at += count
            entries = [StepEntry(i, [0] * n, []) for i, n in enumerate(lens)]
            return pack_step(entries, list(firsts), list(range(len(lens))), [rows], device)

        for name, lens, firsts in (("prefill", [prompt_tokens], [0]), ("decode", [1] * batch, [context] * batch)):
            ctx = context_for(lens, firsts)
            tokens = sum(lens)
            cache = LayerCache(CacheNeed("pages"), True, None, ctx.block_tables[0], page, None, planes)
            causal = sum(f + i + 1 for n, f in zip(lens, firsts) for i in range(n))
            width = -(-(2 * H * D + 2 * G * D + G * VD) // 8) * 8
            rows = torch.randn(tokens, width, device=device).to(bf16)
            mixed = torch.empty(tokens, H * VD, dtype=bf16, device=device)
            store_ms = timed(lambda: ops.diff_store(rows, 2 * H * D, 2 * H * D + 2 * G * D, ones, ones, 1e-5, inv_freq, extra["rot"], ctx.positions, ctx.token_seq, cache, H, G, D, VD))
            ms = timed(lambda: ops.diff_attention(rows, ctx.positions, ctx.token_seq, cache, mixed, H, G, D, VD, D ** -0.5, 0.4, 1e-5, 0.5, batch=ctx))
            qkv = torch.randn(tokens, (LH + 2 * LG) * D, device=device).to(bf16)
            plain = torch.empty(tokens, LH * D, dtype=bf16, device=device)
            like_ms = timed(lambda: ops.paged_attention(qkv, like_pages, ctx.positions, ctx.token_seq, ctx.block_tables[0], plain, LH, LG, D, page, 0, D ** -0.5, batch=ctx))
            x = torch.randn(tokens, W, device=device).to(bf16)
            ids = torch.empty(tokens, top, dtype=torch.int32, device=device)
            weights = torch.empty(tokens, top, device=device)
            route_ms = timed(lambda: ops.moe_route(x, router, None, ids, weights, extra["groups"][0], extra["groups"][1], 2.0))
            routed = torch.empty(tokens, W, dtype=bf16, device=device)
            experts_ms = timed(lambda: ops.moe_experts(x, gate_up, down, ids, weights, None, routed, "silu", batch=ctx))
            act = torch.empty(tokens, top * F, dtype=bf16, device=device)
            stream = torch.zeros(tokens, W, device=device)

            def like_feed_forward():
                ops.linear_gated(x, like_gate_up, act)
                ops.linear_accumulate(act, like_down, stream)

            like_ff_ms = timed(like_feed_forward)
            if name == "prefill":
                flops, like_flops = causal * H * 2 * (2.0 * D + 2.0 * VD), causal * LH * 4.0 * D
                ff_flops = tokens * top * 3 * 2.0 * F * W
                out["attention_prefill"] = {"ms": ms, "tflops": flops / ms / 1e9, "frac": flops / (ms / 1e3) / (peak["bf16_tflops"] * 1e12), "store_ms": store_ms,
                                            "like_ms": like_ms, "like_tflops": like_flops / like_ms / 1e9, "like_frac": like_flops / (like_ms / 1e3) / (peak["bf16_tflops"] * 1e12)}
                out["experts_prefill"] = {"ms": experts_ms, "route_ms": route_ms, "tflops": ff_flops / experts_ms / 1e9, "frac": ff_flops / (experts_ms / 1e3) / (peak["bf16_tflops"] * 1e12),
                                          "like_ms": like_ff_ms, "like_tflops": ff_flops / like_ff_ms / 1e9, "like_frac": ff_flops / (like_ff_ms / 1e3) / (peak["bf16_tflops"] * 1e12)}
            else:
                moved, like_moved = causal * G * (2 * D + VD) * 2.0, causal * LG * 2 * D * 2.0
                chosen = len(torch.unique(ids))
                ff_moved, like_ff_moved = chosen * 3.0 * F * W * 2.0, top * 3.0 * F * W * 2.0
                out["attention_decode"] = {"ms": ms, "gbs": moved / ms / 1e6, "frac": moved / (ms / 1e3) / 1e9 / peak["hbm_gbs"], "store_ms": store_ms,
                                           "like_ms": like_ms, "like_gbs": like_moved / like_ms / 1e6, "like_frac": like_moved / (like_ms / 1e3) / 1e9 / peak["hbm_gbs"]}
                out["experts_decode"] = {"ms": experts_ms, "route_ms": route_ms, "experts_read": chosen, "gbs": ff_moved / experts_ms / 1e6, "frac": ff_moved / (experts_ms / 1e3) / 1e9 / peak["hbm_gbs"],
                                         "like_ms": like_ff_ms, "like_gbs": like_ff_moved / like_ff_ms / 1e6, "like_frac": like_ff_moved / (like_ff_ms / 1e3) / 1e9 / peak["hbm_gbs"]}
            y = torch.randn(tokens, W, device=device).to(bf16)
            normed = torch.empty(tokens, W, dtype=bf16, device=device)
            norm_ms = timed(lambda: ops.branch_norm(stream, y, torch.ones(W, device=device), torch.ones(W, device=device), normed, 1e-5, True))
            like_norm_ms = timed(lambda: ops.add_rmsnorm(stream, y, torch.ones(W, device=device), 1e-5, normed))
            norm_moved = tokens * W * (2 + 4 + 4 + 2.0)
            out[f"norms_{name}"] = {"ms": norm_ms, "gbs": norm_moved / norm_ms / 1e6, "frac": norm_moved / (norm_ms / 1e3) / 1e9 / peak["hbm_gbs"],
                                    "like_ms": like_norm_ms, "like_gbs": norm_moved / like_norm_ms / 1e6, "like_frac": norm_moved / (like_norm_ms / 1e3) / 1e9 / peak["hbm_gbs"]}
        return out

    def kilurax_kernel_numbers(size: dict, extra: dict, like: dict) -> dict:
        """Kilurax's own kernels alone against their rooflines, beside the like kernels of the closest designs at the same sizes: the recurrence without
        the correction beside Zirutar's delta rule (the same kernel, one more dot product per row), each mixer's preparation beside the delta rule's, the
        experts that read their token times its score beside experts whose output is weighed, the grouped norm beside the ungrouped one, and the small
        per-token kernels (convolution in front of a sublayer, embedding with the token before, biases + rotation + cache write) beside the add + norm."""
        W, page, bf16 = size["width"], 64, torch.bfloat16
        E, top, F = extra["experts"], extra["top"], extra["expert_ff"]
        out = {}
        gate_up = (torch.randn(E, 2 * F, W, device=device) * W ** -0.5).to(bf16)
        down = (torch.randn(E, W, F, device=device) * F ** -0.5).to(bf16)
        router = torch.randn(E, W, device=device) * W ** -0.5
        left = extra["left"]
        H, G, D, VD = left["heads"], left["kv_heads"], left["dim"], left["vdim"]
        pages_needed = -(-(context + 1) // page) * batch + -(-prompt_tokens // page)
        pages = torch.randn(pages_needed, 2, G, page, D, device=device).to(bf16) if D == VD else None
        planes = () if D == VD else (torch.randn(pages_needed, G, page, D, device=device).to(bf16), torch.randn(pages_needed, G, page, VD, device=device).to(bf16))
        inv_freq = torch.tensor([10000.0 ** (-2.0 * i / left["rot"]) for i in range(left["rot"] // 2)], dtype=torch.float32, device=device)
        biases = tuple(torch.randn(n, device=device) for n in (H * D, G * D, G * VD))

        def context_for(lens, firsts):
            table_width = size["positions"] // page
            rows, at = [], 0
            for n, f in zip(lens, firsts):
                count = -(-(f + n) // page)
                rows.append(list(range(at, at + count)) + [-1] * (table_width - count))
                at += count
            entries = [StepEntry(i, [0] * n, []) for i, n in enumerate(lens)]
            return pack_step(entries, list(firsts), list(range(len(lens))), [rows], device)

        recurrences = {"state_space": (extra["right"]["heads"], extra["right"]["groups"], extra["right"]["state"], extra["right"]["vdim"], True),
                       "hgrn2": (extra["hgrn2"]["heads"], extra["hgrn2"]["heads"], extra["hgrn2"]["dim"], extra["hgrn2"]["vdim"], True),
                       "delta_per_head": (extra["delta"]["heads"], extra["delta"]["kv_heads"], extra["delta"]["dim"], extra["delta"]["vdim"], False),
                       "like_delta_per_channel": (like["delta_heads"], like["delta_heads"], like["delta_dim"], like["delta_vdim"], False)}
        for name, lens, firsts in (("prefill", [prompt_tokens], [0]), ("decode", [1] * batch, [context] * batch)):
            ctx = context_for(lens, firsts)
            tokens = sum(lens)
            for key, (heads, kv, dim, vdim, plain) in recurrences.items():
                words, _ = ops.delta_state_words(heads, dim, vdim, 0, 1)
                state = torch.zeros(len(lens), words, device=device)
                prep = torch.rand(tokens, 2 * kv * dim + heads * (vdim + 1 + dim), device=device) * 0.5
                read = torch.empty(tokens, heads * vdim, device=device)
                ms = timed(lambda: ops.delta_rule(prep, state, ctx, read, heads, kv, dim, vdim, plain=plain))
                moved = prep.numel() * 4.0 + read.numel() * 4.0 + 2.0 * state.numel() * 4.0
                out[f"recurrence_{key}_{name}"] = {"ms": ms, "gbs": moved / ms / 1e6, "frac": moved / (ms / 1e3) / 1e9 / peak["hbm_gbs"], "heads": heads, "dim": dim, "vdim": vdim}
            # each mixer's preparation (32-bit rows for the recurrence) and what follows the recurrence
            r = extra["right"]
            inner, gn = r["heads"] * r["vdim"], r["groups"] * r["state"]
            rows = torch.randn(tokens, 2 * inner + 2 * gn + r["heads"], device=device).to(bf16)
            words, conv_at = ops.delta_state_words(r["heads"], r["state"], r["vdim"], inner + 2 * gn, r["conv"])
            state = torch.zeros(len(lens), words, device=device)
            prep = torch.empty(tokens, 2 * gn + inner + r["heads"] + r["heads"] * r["state"], device=device)
            taps, conv_bias = torch.randn(inner + 2 * gn, r["conv"], device=device), torch.randn(inner + 2 * gn, device=device)
            per_head = torch.randn(r["heads"], device=device)
            ms = timed(lambda: ops.ssd_prepare(rows, taps, conv_bias, per_head, per_head, state, conv_at, ctx, prep, r["heads"], r["groups"], r["state"], r["vdim"]))
            moved = rows.numel() * 2.0 + prep.numel() * 4.0
            out[f"prepare_state_space_{name}"] = {"ms": ms, "gbs": moved / ms / 1e6, "frac": moved / (ms / 1e3) / 1e9 / peak["hbm_gbs"]}
            read, gated = torch.randn(tokens, inner, device=device), torch.empty(tokens, inner, dtype=bf16, device=device)
            ms = timed(lambda: ops.ssd_finish(read, prep, 2 * gn, rows, per_head, torch.ones(inner, device=device), gated, 1e-5, r["heads"], r["vdim"], r["norm_groups"]))
            moved = inner * tokens * (4.0 + 4.0 + 2.0 + 2.0)
            out[f"finish_state_space_{name}"] = {"ms": ms, "gbs": moved / ms / 1e6, "frac": moved / (ms / 1e3) / 1e9 / peak["hbm_gbs"]}
            h = extra["hgrn2"]
            rows = torch.randn(tokens, 2 * h["heads"] * h["dim"] + h["heads"] * h["vdim"], device=device).to(bf16)
            prep = torch.empty(tokens, 3 * h["heads"] * h["dim"] + h["heads"] * h["vdim"] + h["heads"], device=device)
            lower = torch.rand(h["heads"] * h["dim"], device=device)
            ms = timed(lambda: ops.hgrn2_prepare(rows, lower, lower, prep, h["heads"], h["dim"], h["vdim"]))
            moved = rows.numel() * 2.0 + prep.numel() * 4.0
            out[f"prepare_hgrn2_{name}"] = {"ms": ms, "gbs": moved / ms / 1e6, "frac": moved / (ms / 1e3) / 1e9 / peak["hbm_gbs"]}
            for key, (heads, kv, dim, vdim, per) in {"delta_per_head": (extra["delta"]["heads"], extra["delta"]["kv_heads"], extra["delta"]["dim"], extra["delta"]["vdim"], True),
                                                     "like_delta_per_channel": (like["delta_heads"], like["delta_heads"], like["delta_dim"], like["delta_vdim"], False)}.items():
                channels = 2 * kv * dim + heads * vdim
                rows = torch.randn(tokens, channels + 2 * heads, device=device).to(bf16)
                decay_in = rows[:, channels + heads :] if per else torch.randn(tokens, heads * dim, device=device).to(bf16)
                words, conv_at = ops.delta_state_words(heads, dim, vdim, channels, 4)
                state = torch.zeros(len(lens), words, device=device)
                prep = torch.empty(tokens, channels + heads + heads * dim, device=device)
                taps = torch.randn(channels, 4, device=device)
                a_log, dt_bias = torch.randn(heads, device=device), torch.randn(heads if per else heads * dim, device=device)
                ms = timed(lambda: ops.delta_prepare(rows, channels, decay_in, taps, a_log, dt_bias, state, conv_at, ctx, prep, heads, kv, dim, vdim, 1e-6, dim ** -0.5, decay_per_head=per))
                moved = rows.numel() * 2.0 + prep.numel() * 4.0 + (0 if per else decay_in.numel() * 2.0)
                out[f"prepare_{key}_{name}"] = {"ms": ms, "gbs": moved / ms / 1e6, "frac": moved / (ms / 1e3) / 1e9 / peak["hbm_gbs"]}
            # experts: the score on what the expert reads, beside the weight on what it returns
            x = torch.randn(tokens, W, device=device).to(bf16)
            ids = torch.empty(tokens, top, dtype=torch.int32, device=device)
            weights = torch.empty(tokens, top, device=device)
            route_ms = timed(lambda: ops.moe_route(x, router, None, ids, weights, 1, 1, 1.0, normalize=False))
            routed = torch.empty(tokens, W, dtype=bf16, device=device)
            experts_ms = timed(lambda: ops.moe_experts(x, gate_up, down, ids, weights, None, routed, "silu", batch=ctx, weight_input=True))
            like_ms = timed(lambda: ops.moe_experts(x, gate_up, down, ids, weights, None, routed, "silu", batch=ctx))
            if name == "prefill":
                ff_flops = tokens * top * 3 * 2.0 * F * W
                out["experts_prefill"] = {"ms": experts_ms, "route_ms": route_ms, "tflops": ff_flops / experts_ms / 1e9, "frac": ff_flops / (experts_ms / 1e3) / (peak["bf16_tflops"] * 1e12),
                                          "like_ms": like_ms, "like_frac": ff_flops / (like_ms / 1e3) / (peak["bf16_tflops"] * 1e12)}
            else:
                ff_moved = len(torch.unique(ids)) * 3.0 * F * W * 2.0
                out["experts_decode"] = {"ms": experts_ms, "route_ms": route_ms, "gbs": ff_moved / experts_ms / 1e6, "frac": ff_moved / (experts_ms / 1e3) / 1e9 / peak["hbm_gbs"],
                                         "like_ms": like_ms, "like_frac": ff_moved / (like_ms / 1e3) / 1e9 / peak["hbm_gbs"]}
            # row-wise kernels: the grouped norm around a branch, the convolution in front of a sublayer, the embedding, the cache write
            stream, y = torch.zeros(tokens, W, device=device), torch.randn(tokens, W, device=device).to(bf16)
            normed, ones = torch.empty(tokens, W, dtype=bf16, device=device), torch.ones(W, device=device)
            norm_ms = timed(lambda: ops.branch_norm(stream, y, ones, ones, normed, 1e-5, False, groups=extra["norm_groups"]))
            like_norm_ms = timed(lambda: ops.branch_norm(stream, y, ones, ones, normed, 1e-5, True))
            norm_moved = tokens * W * (2 + 4 + 4 + 2.0)
            out[f"norms_{name}"] = {"ms": norm_ms, "gbs": norm_moved / norm_ms / 1e6, "frac": norm_moved / (norm_ms / 1e3) / 1e9 / peak["hbm_gbs"],
                                    "like_ms": like_norm_ms, "like_frac": norm_moved / (like_norm_ms / 1e3) / 1e9 / peak["hbm_gbs"]}
            kept = torch.zeros(len(lens), (extra["taps"] - 1) * W, device=device)
            conv_taps, filtered = torch.randn(W, extra["taps"], device=device), torch.empty(tokens, W, dtype=bf16, device=device)
            conv_ms = timed(lambda: ops.conv_residual(y, conv_taps, kept, 0, ctx, filtered))
            out[f"input_convolution_{name}"] = {"ms": conv_ms, "gbs": tokens * W * 4.0 / conv_ms / 1e6, "frac": tokens * W * 4.0 / (conv_ms / 1e3) / 1e9 / peak["hbm_gbs"]}
            table, pairs = torch.randn(size["vocab"], W, device=device).to(bf16), torch.randn(65522, W, device=device).to(bf16)
            word = torch.zeros(len(lens), 1, device=device)
            embed_ms = timed(lambda: ops.pair_embedding(table, pairs, ctx, word, 0, ones, 1e-5, 3.0, stream, 65521, 31, 7, extra["norm_groups"]))
            out[f"pair_embedding_{name}"] = {"ms": embed_ms, "gbs": tokens * W * 8.0 / embed_ms / 1e6, "frac": tokens * W * 8.0 / (embed_ms / 1e3) / 1e9 / peak["hbm_gbs"]}
            cache = LayerCache(CacheNeed("pages"), True, pages, ctx.block_tables[0], page, None, planes)
            qkv = torch.randn(tokens, (H + G) * D + G * VD, device=device).to(bf16)
            store_ms = timed(lambda: ops.rotary_store_planes(qkv, H * D, (H + G) * D, biases, inv_freq, left["rot"], ctx.positions, ctx.token_seq, cache, H, G, D, VD))
            like_store_ms = timed(lambda: ops.store_kv_planes(qkv, H * D, (H + G) * D, ctx.positions, ctx.token_seq, cache, G, D, VD))
            mixed = torch.empty(tokens, H * VD, dtype=bf16, device=device)
            ms = timed(lambda: ops.mixed_heads_attention(qkv, -1, ctx.positions, ctx.token_seq, cache, None, None, mixed, H, G, D, VD, 0, D ** -0.5, batch=ctx))
            causal = sum(f + i + 1 for n, f in zip(lens, firsts) for i in range(n))
            if name == "prefill":
                flops = causal * H * 2.0 * (D + VD)
                out["attention_prefill"] = {"ms": ms, "tflops": flops / ms / 1e9, "frac": flops / (ms / 1e3) / (peak["bf16_tflops"] * 1e12), "store_ms": store_ms, "like_store_ms": like_store_ms}
            else:
                moved = causal * G * (D + VD) * 2.0
                out["attention_decode"] = {"ms": ms, "gbs": moved / ms / 1e6, "frac": moved / (ms / 1e3) / 1e9 / peak["hbm_gbs"], "store_ms": store_ms, "like_store_ms": like_store_ms}
        return out

    results = {}
    which = args.designs
    with ClockSampler() as clocks:
        for key, size in DESIGN_SIZES.items():
            marutar, llama = design_configs(size)
            base = Path(tempfile.gettempdir()) / f"tlie_b200_designs_{os.getuid()}_{key}"
            if which == "kilurax":
                pair = (("kilurax", kilurax_config(size, KILURAX_SIZES[key])), ("redasun", redasun_config(size, REDASUN_SIZES[key])))
            elif which == "redasun":
                pair = (("redasun", redasun_config(size, REDASUN_SIZES[key])), ("llama", llama))
            else:
                pair = (("marutar", marutar), ("llama", llama)) if which == "marutar" else (("zirutar", zirutar_config(size, ZIRUTAR_SIZES[key])), ("marutar", marutar))
            folders = {}
            for name, config in pair:
                folders[name] = base / name
                if not (folders[name] / "model.safetensors").exists():
                    write_random_model(folders[name], config, seed=0)
            results[key] = {name: model_numbers(folders[name]) for name, _ in pair}
            if which == "kilurax":
                results[key]["kernels"] = kilurax_kernel_numbers(size, KILURAX_SIZES[key], ZIRUTAR_SIZES[key])
            elif which == "redasun":
                results[key]["kernels"] = redasun_kernel_numbers(size, REDASUN_SIZES[key])
            else:
                results[key]["kernels"] = kernel_numbers(size) if which == "marutar" else zirutar_kernel_numbers(size, ZIRUTAR_SIZES[key])
            results[key]["sizes"] = {k: v for k, v in size.items() if k != "pattern"} | {"pattern": "/".join(size["pattern"])}
            if which == "redasun":
                results[key]["sizes"] = {k: v for k, v in size.items() if k in ("width", "ff", "vocab", "layers")} | {k: (list(v) if isinstance(v, tuple) else v) for k, v in REDASUN_SIZES[key].items()}
            if which == "kilurax":
                results[key]["sizes"] = {k: v for k, v in size.items() if k in ("width", "vocab", "layers")} | {k: (list(v) if isinstance(v, tuple) else v) for k, v in KILURAX_SIZES[key].items()}
            if which == "zirutar":
                results[key]["sizes"] |= {k: v for k, v in ZIRUTAR_SIZES[key].items() if k != "pattern"} | {"zirutar_pattern": "/".join(ZIRUTAR_SIZES[key]["pattern"])}
    names = {"marutar": "Marutar beside the Llama decoder", "zirutar": "Zirutar beside Marutar", "redasun": "Redasun beside the Llama decoder",
             "kilurax": "Kilurax beside Redasun"}[which]
    return {"metric": f"prompt and decode throughput of {names} at equal sizes", "unit": "tokens/s", "n_gpus": 1, "dtype": "bf16",
            "data": "synthetic (random weights, uniform random token ids)", "impl": "engine", "higher_is_better": True,
            "config": {"prompt_tokens": prompt_tokens, "decode_context": context, "decode_batch": batch, "decode_steps": steps, "page_size": 64, "peaks": peak_kind,
                       "l2": "a buffer larger than L2 is written before every timed launch"},
            "peaks": peak, "designs": results, "clocks": clocks.summary()}


def run_reference(args) -> dict:
    """The unmodified reference on the same metric: TinyLlama 1.1B, 1,024-token prompts, greedy decoding, float16."""
    sys.path.insert(0, str(ROOT / "baseline"))
    import reference_arm

    try:
        if args.config != "tinyllama" or (args.layers or 22) != 22:
            raise reference_arm.Unavailable("the reference runs the TinyLlama-1.1B configuration with all 22 layers only (src/model_config.cpp:54-76)")
        chosen = CONFIGS["tinyllama"]
        if args.batch > 64:
            raise reference_arm.Unavailable("the reference's batched step takes at most 64 rows (src/cuda/model.cu:344-348)")
        warmup = max(args.warmup, 3)
        folder = model_folder("tinyllama", chosen["shapes"], 22)
        # the other batch sizes only on request: the reference feeds a prompt one position per step, three minutes for 64 requests
        batches = [args.batch] + [b for b in (1, 64) if b != args.batch and args.reference_points]
        with ClockSampler() as clocks:
            records = reference_arm.run(folder, chosen["prompt_tokens"], warmup, args.steps, batches)
    except reference_arm.Unavailable as reason:
        return {"impl": "reference", "unavailable": str(reason)}
    main_record = records[args.batch]
    peak, peak_kind = peaks()
    first_context = chosen["prompt_tokens"] + warmup
    step_bytes = decode_bytes(chosen["shapes"], 22, args.batch, first_context + (args.steps + 1) / 2.0)
    achieved = step_bytes / (main_record["device_ms_per_step"] / 1e3) / 1e9
    vocab = chosen["shapes"]["vocab_size"]
    return {
        "metric": metric_name(args, chosen),
        "value": args.batch * 1e3 / main_record["device_ms_per_step"], "unit": "tokens/s", "n_gpus": 1, "steps": args.steps, "warmup": warmup,
        "ms_per_step": main_record["device_ms_per_step"], "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "fp16",
        "data": "synthetic (the engine arm's random weights as float16, uniform random token ids)", "impl": "reference",
        "config": config_record(args, chosen, 22, first_context, peak_kind),
        # a whole step of the reference's API: token ids in from the host, float16 logits of every row out and greedy on the host
        "e2e": {"value": args.batch * 1e3 / main_record["wall_ms_per_step"], "unit": "tokens/s", "h2d_bytes_per_step": args.batch * 4,
                "d2h_bytes_per_step": args.batch * vocab * 2},
        "gpu_launches": None, "prefill": None,
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak["hbm_gbs"], "unit": "GB/s", "frac": achieved / peak["hbm_gbs"], "bytes_per_step": step_bytes},
        "points": {f"decode_b{b}": b * 1e3 / records[b]["device_ms_per_step"] for b in records if b in (1, 64)},
        "clocks": clocks.summary(),
    }


def main() -> int:
    parser = argparse.ArgumentParser()
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=256)
    parser.add_argument("--warmup", type=int, default=3)
    parser.add_argument("--batch", type=int, default=8)
    parser.add_argument("--config", default="tinyllama", choices=sorted(CONFIGS), help="whose layer sizes to run (random weights)")
    parser.add_argument("--layers", type=int, default=0, help="layers to run (default: all 22 of tinyllama, 8 of the 32 of the larger shapes)")
    parser.add_argument("--prefill-samples", type=int, default=5)
    parser.add_argument("--impl", default="engine", choices=["engine", "reference"])
    parser.add_argument("--reference-points", action="store_true", help="with --impl reference: also time batch 1 and 64 (minutes)")
    parser.add_argument("--sections", default="decode,e2e,prefill,points,mixed", help="which measurements to take (fewer for profiling runs; `mixed` adds requests of mixed length through the scheduler)")
    parser.add_argument("--designs", nargs="?", const="marutar", default=None, choices=["marutar", "zirutar", "redasun", "kilurax"],
                        help="instead of the headline workload: another design beside the closest existing one at equal sizes (prompt and decode throughput through "
                             "the engine, and the design's own kernels against their rooflines): Marutar beside the Llama decoder (the default), Zirutar beside Marutar, Redasun beside the Llama decoder, or Kilurax beside Redasun")
    args = parser.parse_args()
    if args.gpus != 1:
        print(f"bench.py measures one GPU only: this engine is single-GPU by design (asked for {args.gpus})")
        return 2
    if args.designs:
        print(json.dumps(run_designs(args)))
        return 0
    print(json.dumps(run_reference(args) if args.impl == "reference" else run_engine(args)))
    return 0


if __name__ == "__main__":
    sys.exit(main())
