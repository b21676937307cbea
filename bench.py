#!/usr/bin/env python3
"""Decode and prefill throughput of the engine at Qwen3 layer sizes with random weights.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--batch 8] [--impl ours|reference] [--model 8b|0.6b|32b]

One step is one decode step of the whole batch.  The default run: 36 layers of the 8B sizes, bfloat16, a batch of 8
sequences with 1,024-token random prompts in a 4,096-token context, W untimed then K timed decode steps replayed from
CUDA graphs and timed with CUDA events.  One JSON line is printed:

  value      decoded tokens a second, timed on the device (tokens stay on the device)
  e2e        the same through ``generate`` (host token lists in, host token lists out; every step copies its input
             ids from pinned host memory and reads the sampled ids back): one call that runs the prompts, W untimed
             decode steps and the K timed ones, by the loop's own clock around each step (``value_all_steps``: over
             all W + K; the first dozen steps after a prompt step run at the clocks the prompt left)
  prefill    one prompt of 2,048 tokens: tokens a second, and flops / time / peak
  roofline   decode: (every weight once + the live sequences' cache) / step time, against the HBM peak
  points     decode tokens a second at batch 1 and 64 with their roofline fractions, prefill of 4,096 tokens (the context),
             and the benchmark's two other workloads (left out with --skip-other-models): Qwen3-0.6B sizes, 16 prompts
             with lengths uniform in [1, 2048] in one prefill step, then 128 decode steps; Qwen3-32B sizes, all 64
             layers, a 2,048-token prefill and decode at batch 1, 8 and 16 from 1,024-token prompts

``--model 0.6b`` or ``--model 32b`` runs one of those workloads alone and prints a line of its own.
``--impl reference`` runs kishida/questwend itself (built by baseline/build_reference.py into baseline/_ref/) on the
same sizes: it holds one sequence, so the batch is run as that many sequences one after the other.

Peaks come from MEASURED_PEAKS.json beside this file when it is there ("of measured"),
else from the fallback figures 6.65 TB/s and 1.59 PFLOP/s ("of fallback").  Every decode
step reads more than 15 GB of weights, far more than the 126 MB L2, so no L2 flush is needed
between timed steps (config.l2 says so).
"""
from __future__ import annotations

import argparse
import gc
import json
import os
import shutil
import statistics
import subprocess
import sys
import tempfile
import threading

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

QWEN3_8B = {                     # the layer sizes of Qwen3-8B: the model this benchmark is quoted on
    "architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3",
    "num_hidden_layers": 36, "hidden_size": 4096, "num_attention_heads": 32, "num_key_value_heads": 8,
    "head_dim": 128, "intermediate_size": 12288, "vocab_size": 151936, "rope_theta": 1e6,
    "rms_norm_eps": 1e-6, "tie_word_embeddings": False, "max_position_embeddings": 4096,
}
QWEN3_06B = dict(QWEN3_8B, num_hidden_layers=28, hidden_size=1024, num_attention_heads=16, num_key_value_heads=8,
                 intermediate_size=3072, tie_word_embeddings=True)
QWEN3_32B = dict(QWEN3_8B, num_hidden_layers=64, hidden_size=5120, num_attention_heads=64, num_key_value_heads=8,
                 intermediate_size=25600)
MODELS = {"8b": QWEN3_8B, "0.6b": QWEN3_06B, "32b": QWEN3_32B}


def movudra_sizes(width=2048, repeats=2, window=4096, vocab=32768):
    """A Movudra configuration at sizes that resemble real layers: per repeat one gated delta layer (16 heads of
    128 x 128) with a dense feed-forward of 4 x width, one latent attention layer (16 heads of 128 + 64, latent 512,
    query latent 1,536) and one Mamba-2 layer (inner 2 x width in heads of 64, state 128, 8 groups), the last two with
    64 routed experts of 1,408 of which a token uses 6."""
    moe = {"kind": "moe", "expert": {"ff": 1408}, "router": {"experts": 64, "top": 6}}
    delta = {"type": "channel_delta", "mixer": {"conv": 4, "dim": 128, "heads": width // 128, "kv_heads": width // 128, "vdim": 128},
             "mlp": {"kind": "dense", "ff": 4 * width}}
    latent = {"type": "latent_attention", "mlp": moe,
              "mixer": {"dim": 128, "heads": width // 128, "kv_rank": 512, "q_rank": 1536, "rot_dim": 64, "vdim": 128,
                        "scale": 192 ** -0.5, "mask": {"size": window},
                        "rot": {"base": 10000.0, "dims": 64, "scaling": {"factor": 4.0, "fast": 32.0, "original": 4096, "slow": 1.0}}}}
    mamba = {"type": "mamba2", "mlp": moe,
             "mixer": {"conv": 4, "groups": 8, "heads": 2 * width // 64, "norm_groups": 8, "state": 128, "vdim": 64}}
    return {"architecture": "Movudra", "layers": [delta, latent, mamba] * repeats, "norm": {"eps": 1e-5},
            "vocab": vocab, "width": width}


def roritar_sizes(width=2048, repeats=2, window=1024, pool=16, vocab=32768):
    """A Roritar configuration at sizes that resemble real layers: per repeat two recurrent layers (2,560 channels in 10
    blocks of 256, 4 taps) and one attention layer (16 heads of 128 over 4 key/value heads, values of 128, a window of
    1,024 tokens and blocks of 16, half of each head rotated), each with a dense feed-forward of 4 x width."""
    mlp = {"kind": "dense", "ff": 4 * width}
    rec = {"type": "rglru", "mixer": {"blocks": 10, "conv": 4, "width": width * 5 // 4}, "mlp": mlp}
    att = {"type": "attention", "mlp": mlp,
           "mixer": {"dim": 128, "heads": width // 128, "kv_heads": width // 512, "vdim": 128, "scale": 128 ** -0.5,
                     "mask": {"size": window, "pool": pool}, "rot": {"base": 10000.0, "dims": 64}}}
    return {"architecture": "Roritar", "layers": [rec, rec, att] * repeats, "norm": {"eps": 1e-5}, "vocab": vocab, "width": width,
            "logit_scale": 1.0, "logit_softcap": 30.0}


def punolix_sizes(width=2048, repeats=2, chunk=1024, vocab=32768):
    """A Punolix configuration at sizes that resemble real layers: per repeat a differential attention layer (16 heads with
    two score maps of 64 over 4 key/value heads, values of 128, scores capped at 50), a layer with two mixers side by side
    (attention inside chunks of 1,024 positions, 16 heads of 128 over 4 key/value heads behind a convolution of 4 taps,
    beside gated linear attention with 4 heads of 256 x 512 and a decay projection of rank 16) and another differential
    layer, each with a gated feed-forward of 3 x width."""
    mlp = {"kind": "dense", "ff": 3 * width}
    diff = {"type": "attention", "mlp": mlp,
            "mixer": {"diff": 0.8, "dim": 64, "heads": width // 128, "kv_heads": width // 512, "vdim": 128, "scale": 64 ** -0.5,
                      "softcap": 50.0, "rot": {"base": 10000.0, "dims": 64}}}
    left = {"conv": 4, "dim": 128, "heads": width // 128, "kv_heads": width // 512, "vdim": 128, "scale": 128 ** -0.5,
            "mask": {"size": chunk},
            "rot": {"base": 500000.0, "dims": 128, "scaling": {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 8192}}}
    right = {"dim": width // 8, "heads": 4, "tau": 16.0, "vdim": width // 4}
    pair = {"type": "parallel", "mlp": mlp, "mixer": {"left": left, "right": right, "left_scale": 1.0, "right_scale": 1.0}}
    return {"architecture": "Punolix", "embedding": {"scale": 1.0}, "layers": [diff, pair, diff] * repeats, "norm": {"eps": 1e-5},
            "residual_mult": 0.7, "vocab": vocab, "width": width}


def sagupel_sizes(width=2048, repeats=2, window=1024, vocab=32768):
    """A Sagupel configuration at sizes that resemble real layers: per repeat a retention layer (16 heads of 128 x 128, all
    of q and k turned), a layer with two mixers side by side (attention with capped scores, a number per head, mixed heads
    and a gate per head, 16 heads of 128 over 4 key/value heads, beside the gated delta rule with a decay per head, 16
    heads of 128 x 128 over 4 query/key heads, 4 taps) and an attention layer over a window of 1,024 positions with a
    distance bias and a sink (16 heads of 128 over 4 key/value heads), each behind an input convolution of 3 taps and
    with a clamped gated feed-forward of 3 x width."""
    mlp = {"kind": "dense", "ff": 3 * width, "limit": 7.0}
    heads = width // 128
    ret = {"type": "retention", "mlp": mlp,
           "mixer": {"decay": [1.0 - 2.0 ** (-5 - 3 * h / heads) for h in range(heads)], "dim": 128, "heads": heads, "vdim": 128,
                     "rot": {"base": 500000.0, "dims": 128}}}
    left = {"dim": 128, "heads": heads, "kv_heads": width // 512, "vdim": 128, "scale": 128 ** -0.5, "softcap": 25.0,
            "rot": {"base": 10000.0, "dims": 64, "scaling": {"factor": 8.0}}}
    right = {"conv": 4, "dim": 128, "heads": heads, "kv_heads": width // 512, "vdim": 128}
    pair = {"type": "parallel", "mlp": mlp, "mixer": {"left": left, "right": right}}
    win = {"type": "attention", "mlp": mlp,
           "mixer": {"dim": 128, "heads": heads, "kv_heads": width // 512, "vdim": 128, "scale": 128 ** -0.5, "mask": {"size": window}}}
    return {"architecture": "Sagupel", "canon": {"taps": 3}, "layers": [ret, pair, win] * repeats, "norm": {"eps": 1e-5},
            "postln_alpha": 1.5, "vocab": vocab, "width": width}


def qwen3_beside(width=2048, layers=6, vocab=32768):
    """The closest model the library had, at the same width, depth and vocabulary: Qwen3 layers with 16 heads of 128
    (8 key/value heads) and a gated feed-forward of 3 x width."""
    return dict(QWEN3_8B, num_hidden_layers=layers, hidden_size=width, num_attention_heads=width // 128,
                num_key_value_heads=width // 256, intermediate_size=3 * width, vocab_size=vocab)
N_CTX = 4096
PROMPT_LEN = 1024
PREFILL_TOKENS = 2048
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            d = json.load(f)
        def number(v):                       # a plain number, or an object that holds one under "value"
            return float(v["value"] if isinstance(v, dict) else v)
        peaks = {k: number(d[k]) for k in ("hbm_gbs", "bf16_tflops") if k in d}
        if len(peaks) == 2 and all(v > 0 for v in peaks.values()):
            peaks["bf16_tflops_sustained"] = number(d.get("bf16_tflops_sustained", peaks["bf16_tflops"]))
            return peaks, "measured"
    except Exception:                            # an unreadable file is no reason to lose the run: fall back
        pass
    return dict(FALLBACK_PEAKS), "fallback"


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons while a timed region runs."""
    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.rows = []
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", "0", f"--query-gpu={self.QUERY}",
                                          "--format=csv,noheader,nounits", "-lms", "200"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self) -> dict:
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in self.rows:
            if len(r) < 6:
                continue
            try:
                sm.append(float(r[0]))
                mx.append(float(r[1]))
            except ValueError:
                continue
            for name, v in zip(names, r[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def weight_bytes(engine) -> int:
    """Bytes of every weight a decode step reads once (the embedding table is only gathered from)."""
    total = 0
    for block in engine.model.blocks:
        total += block.mixer.w_qkv.numel() * block.mixer.w_qkv.element_size()
        total += block.mixer.w_o.numel() * block.mixer.w_o.element_size()
        total += block.ffn.w_gate_up.numel() * block.ffn.w_gate_up.element_size()
        total += block.ffn.w_down.numel() * block.ffn.w_down.element_size()
    total += engine.model.head.weight.numel() * engine.model.head.weight.element_size()
    return total


def kv_bytes_per_token(cfg, n_layers, elem=2) -> int:
    return 2 * n_layers * cfg["num_key_value_heads"] * cfg["head_dim"] * elem


def prefill_flops(cfg, n_layers, T) -> float:
    D, Hq, Hkv, hd, F, V = (cfg["hidden_size"], cfg["num_attention_heads"], cfg["num_key_value_heads"],
                            cfg["head_dim"], cfg["intermediate_size"], cfg["vocab_size"])
    per_token = 2 * (D * (Hq + 2 * Hkv) * hd + Hq * hd * D + 3 * D * F)
    attn = 2 * 2 * Hq * hd * (T * (T + 1) / 2)            # causal QK^T and PV
    return n_layers * (T * per_token + attn) + 2 * D * V   # the head runs on one row


def decode_run(engine, torch, batch, warmup, steps, rng, count_launches=False):
    """Prefill `batch` prompts of PROMPT_LEN, then time `steps` graph-replayed decode steps."""
    from questwend_b200.engine.engine import StepEntry
    from questwend_b200.sampling.params import GREEDY
    from questwend_b200.kernels import ops
    V = engine.vocab_size
    prompts = [rng.integers(0, V, PROMPT_LEN).tolist() for _ in range(batch)]
    slots = engine.open_sequences(batch)
    first = []
    for i in range(0, batch, 8):                       # prompts in groups of 8: bounded activation memory
        grp = list(range(i, min(batch, i + 8)))
        lg = engine.step([StepEntry(slots[j], prompts[j], [PROMPT_LEN - 1]) for j in grp])
        first += lg.argmax(-1).tolist()
    runner = engine.decode_runner(batch, GREEDY)
    runner.bind(slots, first, list(range(batch)), 1)
    for _ in range(warmup):
        runner.step()
    torch.cuda.synchronize()
    launches_before = ops.LAUNCHES[0]
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ctx0 = engine.cache.length(slots[0])
    start.record()
    for _ in range(steps):
        runner.step()
    end.record()
    torch.cuda.synchronize()
    ms = start.elapsed_time(end)
    engine.check_kernels()                             # no bounded wait inside a kernel gave up
    ctx1 = engine.cache.length(slots[0])
    per_step = runner.launches_per_step
    engine.close_sequences(slots)
    return {"ms_per_step": ms / steps, "tok_s": batch * steps / (ms / 1e3), "mean_ctx": (ctx0 + ctx1) / 2.0,
            "launches_per_step": per_step, "eager_launches": ops.LAUNCHES[0] - launches_before}


def time_prefill(engine, torch, rng, n_tokens, reps=4) -> float:
    """Median milliseconds of one prompt of ``n_tokens`` in one step (the first run is not counted)."""
    from questwend_b200.engine.engine import StepEntry
    times = []
    for _ in range(reps):
        slot = engine.open_sequences(1)[0]
        prompt = rng.integers(0, engine.vocab_size, n_tokens).tolist()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        a.record()
        engine.step([StepEntry(slot, prompt, [n_tokens - 1])])
        b.record()
        torch.cuda.synchronize()
        times.append(a.elapsed_time(b))
        engine.close_sequences([slot])
    return statistics.median(times[1:])


def make_engine(cfgd, layers, max_batch, tokens_each, n_ctx=N_CTX):
    from questwend_b200.config.registry import config_from_dict
    from questwend_b200.engine.engine import Engine
    d = dict(cfgd)
    d["num_hidden_layers"] = layers
    return Engine.from_config(config_from_dict(d), seed=0, dtype="bfloat16", max_tokens=max_batch * tokens_each,
                              max_seq_len=n_ctx, max_batch=max_batch), d


def release(engine, torch):
    """Give the engine's device memory back (weights, cache, graphs) whoever still holds the object."""
    engine._runners.clear()
    engine.model = engine.cache = engine.unit_caches = None
    gc.collect()
    torch.cuda.empty_cache()


def small_model_workload(torch, np, peaks) -> dict:
    """Qwen3-0.6B sizes: 16 prompts with lengths uniform in [1, 2048] in ONE prefill step, then 128 decode steps."""
    from questwend_b200.engine.engine import StepEntry
    from questwend_b200.sampling.params import GREEDY
    engine, d = make_engine(QWEN3_06B, QWEN3_06B["num_hidden_layers"], 16, 2048 + 256)
    rng = np.random.default_rng(6)
    lengths = rng.integers(1, 2049, 16).tolist()
    out = {}
    pf = []
    for rep in range(3):
        prompts = [rng.integers(0, engine.vocab_size, n).tolist() for n in lengths]
        slots = engine.open_sequences(16)
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        a.record()
        lg = engine.step([StepEntry(s, p, [len(p) - 1]) for s, p in zip(slots, prompts)])
        b.record()
        torch.cuda.synchronize()
        pf.append(a.elapsed_time(b))
        if rep < 2:
            engine.close_sequences(slots)
    pf_ms = min(pf[1:])
    runner = engine.decode_runner(16, GREEDY)
    runner.bind(slots, lg.argmax(-1).tolist(), list(range(16)), 1)
    for _ in range(4):
        runner.step()
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    len0 = sum(engine.cache.length(s) for s in slots)
    a.record()
    for _ in range(128):
        runner.step()
    b.record()
    torch.cuda.synchronize()
    len1 = sum(engine.cache.length(s) for s in slots)
    ms = a.elapsed_time(b) / 128
    step_bytes = weight_bytes(engine) + (len0 + len1) / 2 * kv_bytes_per_token(d, d["num_hidden_layers"])
    T = sum(lengths)
    flops = sum(prefill_flops(d, d["num_hidden_layers"], n) for n in lengths)
    out = {"m06b_b16_decode": 16 / (ms / 1e3), "m06b_b16_decode_ms": ms,
           "m06b_b16_decode_frac": step_bytes / (ms / 1e3) / 1e9 / peaks["hbm_gbs"],
           "m06b_b16_launches_per_step": runner.launches_per_step, "m06b_prefill": T / (pf_ms / 1e3),
           "m06b_prefill_tokens": T, "m06b_prefill_ms": pf_ms,
           "m06b_prefill_frac": flops / (pf_ms / 1e3) / (peaks["bf16_tflops"] * 1e12)}
    engine.close_sequences(slots)
    release(engine, torch)
    return out


def large_model_workload(torch, np, peaks) -> dict:
    """Qwen3-32B sizes, all 64 layers: a 2,048-token prefill, and decode at batch 1, 8 and 16 from 1,024-token prompts."""
    if True:
        engine, d = make_engine(QWEN3_32B, QWEN3_32B["num_hidden_layers"], 16, PROMPT_LEN + 256)
        rng = np.random.default_rng(32)
        out = {"m32b_weights_gb": weight_bytes(engine) / 1e9}
        for b in (1, 8, 16):
            r = decode_run(engine, torch, b, 3, 16, rng)
            step_bytes = weight_bytes(engine) + b * r["mean_ctx"] * kv_bytes_per_token(d, d["num_hidden_layers"])
            out[f"m32b_decode_b{b}"] = r["tok_s"]
            out[f"m32b_decode_b{b}_frac"] = step_bytes / (r["ms_per_step"] / 1e3) / 1e9 / peaks["hbm_gbs"]
        pf_ms = time_prefill(engine, torch, rng, PREFILL_TOKENS, reps=3)
        out["m32b_prefill"] = PREFILL_TOKENS / (pf_ms / 1e3)
        out["m32b_prefill_ms"] = pf_ms
        out["m32b_prefill_frac"] = (prefill_flops(d, d["num_hidden_layers"], PREFILL_TOKENS) / (pf_ms / 1e3)
                                    / (peaks["bf16_tflops"] * 1e12))
        out["m32b_peak_memory_gb"] = torch.cuda.max_memory_allocated() / 1e9
        release(engine, torch)
    return out


def _tensor_bytes(obj, seen) -> int:
    import torch
    total = 0
    for v in vars(obj).values():
        if isinstance(v, torch.Tensor) and v.dim() >= 2 and v.data_ptr() not in seen:
            seen.add(v.data_ptr())
            total += v.numel() * v.element_size()
    return total


def step_weight_bytes(engine, batch: int) -> int:
    """Bytes of the matrices that one decode step of ``batch`` tokens reads at most once each: every bound matrix of the
    mixers and feed-forwards and the head; of routed experts only as many as the batch can choose."""
    seen, total = set(), 0
    for block in engine.model.blocks:
        total += _tensor_bytes(block.mixer, seen)
        ffn = getattr(block, "ffn", None)
        if ffn is None:
            continue
        if hasattr(ffn, "experts"):
            per_expert = (ffn.w_gate_up[0].numel() + ffn.w_down[0].numel()) * ffn.w_down.element_size()
            total += min(ffn.experts, batch * ffn.top) * per_expert + ffn.w_router.numel() * ffn.w_router.element_size()
        else:
            total += _tensor_bytes(ffn, seen)
    return total + engine.model.head.weight.numel() * engine.model.head.weight.element_size()


def time_parts(engine, torch, rng, n_tokens: int, batch: int, prompt: int = 0, reps: int = 5) -> dict:
    """Median microseconds of every layer's mixer and feed-forward alone, in a step of ``batch`` sequences that bring
    ``n_tokens`` tokens each after ``prompt`` cached ones: the parts' own forward calls on the step's context."""
    from questwend_b200.engine.engine import StepEntry
    slots = engine.open_sequences(batch)
    V = engine.vocab_size
    if prompt:
        engine.step([StepEntry(s, rng.integers(0, V, prompt).tolist(), []) for s in slots])
    ctx, _ = engine.build_context([StepEntry(s, rng.integers(0, V, n_tokens).tolist(), []) for s in slots])
    T = ctx.n_tokens
    x = torch.randn(T, engine.plan.hidden_size, device=engine.device).to(engine.dtype)
    for position in engine.model._positions.values():
        position.prepare(ctx)
    out = {}

    def timed(fn):
        times = []
        for _ in range(reps + 1):
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            a.record()
            fn()
            b.record()
            torch.cuda.synchronize()
            times.append(a.elapsed_time(b) * 1e3)
        return round(statistics.median(times[1:]), 1)

    seen = set()
    for i, run in enumerate(engine.model.schedule):
        block = engine.model.blocks[run.layer]
        unit = engine.unit_caches[i]
        mixer = block.mixer
        name = type(mixer).__name__
        if hasattr(mixer, "inner"):                             # a mixer behind an input convolution: named by what it wraps
            inner = mixer.inner
            name = "+".join(type(m).__name__ for m in getattr(inner, "branches", [inner])) + "_behind_conv"
        if name not in seen:
            seen.add(name)
            if getattr(block.mixer, "adds_to_residual", False):
                out[name + "_us"] = timed(lambda: block.mixer.forward(x, ctx, unit, residual=None))
            else:
                out[name + "_us"] = timed(lambda: block.mixer.forward(x, ctx, unit))
        ffn = getattr(block, "ffn", None)
        if ffn is not None and type(ffn).__name__ not in seen:
            seen.add(type(ffn).__name__)
            out[type(ffn).__name__ + "_us"] = timed(lambda: ffn.forward(x, ctx))
    engine.close_sequences(slots)
    return out


def movudra_workload(torch, np, peaks, steps: int, warmup: int, designs=None) -> dict:
    """Prefill and decode of a design at real layer sizes (``movudra_sizes``, ``roritar_sizes``), and of Qwen3 layers of the
    same width, depth and vocabulary (``qwen3_beside``): tokens a second for a 2,048-token prompt and for graph-replayed
    decode steps at batch 1 and 8 after 1,024-token prompts, the decode steps against the HBM roofline of the matrices
    they must read, and the time of every kind of mixer and feed-forward alone in both kinds of step."""
    from questwend_b200.config.registry import config_from_dict
    from questwend_b200.engine.engine import Engine
    out = {}
    for name, cfgd in (designs or (("movudra", movudra_sizes()), ("qwen3_same_size", qwen3_beside()))):
        engine = Engine.from_config(config_from_dict(cfgd), seed=0, dtype="bfloat16", max_tokens=8 * (PROMPT_LEN + 512) + 4096,
                                    max_seq_len=N_CTX, max_batch=9)
        rng = np.random.default_rng(1)
        point = {"parameters": engine.describe()["parameters"], "layers": len(engine.model.blocks)}
        ms = time_prefill(engine, torch, rng, PREFILL_TOKENS)
        point["prefill_2048"] = {"ms": round(ms, 3), "tok_s": round(PREFILL_TOKENS / (ms / 1e3), 1)}
        for batch in (1, 8):
            r = decode_run(engine, torch, batch, warmup, steps, rng)
            wbytes = step_weight_bytes(engine, batch)
            point[f"decode_b{batch}"] = {"ms_per_step": round(r["ms_per_step"], 4), "tok_s": round(r["tok_s"], 1),
                                         "launches_per_step": r["launches_per_step"], "weight_bytes": wbytes,
                                         "hbm_roofline_frac": round(wbytes / (r["ms_per_step"] / 1e3) / (peaks["hbm_gbs"] * 1e9), 3)}
        point["parts_prefill_2048"] = time_parts(engine, torch, rng, PREFILL_TOKENS, 1)
        point["parts_decode_b8"] = time_parts(engine, torch, rng, 1, 8, prompt=PROMPT_LEN)
        out[name] = point
        release(engine, torch)
    return out


def roritar_kernels(torch, np, peaks) -> dict:
    """The Roritar design's own kernels alone at the sizes of ``roritar_sizes``, each beside the like kernel of a model the
    library had, with the bytes or FLOPs it must move and the share of the measured peak that this comes to: the layer
    norms (beside the RMS norms), the recurrence (beside Mamba-2's), its gates, and attention over window and blocks in a
    2,048-token prompt and in decode steps (beside Qwen3's attention over the same number of visible keys)."""
    from questwend_b200.cache.manager import CacheManager
    from questwend_b200.engine.engine import StepEntry, build_step_context
    from questwend_b200.kernels import ops
    from questwend_b200.parts.base import KVSpec, StateSpec
    dev, bf = torch.device("cuda:0"), torch.bfloat16
    hbm, tf = peaks["hbm_gbs"] * 1e9, peaks["bf16_tflops"] * 1e12
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)

    def timed(fn, reps=7):
        times = []
        for _ in range(reps + 3):
            flush.zero_()                                         # L2 holds nothing of the last run
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            fn()
            b.record()
            torch.cuda.synchronize()
            times.append(a.elapsed_time(b) * 1e3)
        return statistics.median(times[3:])

    def point(us, n_bytes=0, flops=0):
        p = {"us": round(us, 1)}
        if n_bytes:
            p.update(gb_s=round(n_bytes / us / 1e3, 1), hbm_frac=round(n_bytes / (us * 1e-6) / hbm, 3))
        if flops:
            p.update(tflops=round(flops / us / 1e6, 1), tensor_frac=round(flops / (us * 1e-6) / tf, 3))
        return p

    out = {}
    T, D, W = 2048, 2048, 2560
    for rows in (T, 8):
        h, y = torch.randn(rows, D, device=dev), torch.randn(rows, D, device=dev)
        w = torch.ones(D, device=dev)
        n = rows * D
        out[f"layer_norm_onto_and_norm_{rows}"] = point(timed(lambda: ops.layernorm(h, w, 1e-5, bf, add=y, add_weight=w, write_sum=True)), 14 * n)
        out[f"rms_norm_onto_then_cast_{rows}"] = point(timed(lambda: ops.rmsnorm_onto(h, y, w, 1e-5, bf)), 14 * n)
        out[f"rms_norm_with_sum_{rows}"] = point(timed(lambda: ops.rmsnorm(h, w, 1e-5, bf, delta=y, write_sum=True)), 14 * n)
    # the recurrences: one prompt of 2,048 tokens, and a step of 8 single tokens
    for rows, B in ((T, 1), (8, 8)):
        cache = CacheManager([(None, (StateSpec((3, W)), StateSpec((W,))), None), (None, (StateSpec((3, 4096 + 2048)), StateSpec((64, 64, 128))), None)],
                             4096, 8, 4096, bf, dev)
        slots = cache.open(B)
        ctx = build_step_context(cache, [StepEntry(s, [0] * (rows // B), []) for s in slots], 10, dev)[0]
        u, r, i = (torch.rand(rows, W, device=dev) for _ in range(3))
        proj, lam, yb = torch.randn(rows, 2 * W, device=dev), torch.randn(W, device=dev), torch.zeros(W, device=dev)
        tail, state = cache.unit_cache(0).state
        out[f"rglru_scan_{rows}"] = point(timed(lambda: ops.rglru_scan(u, r, i, lam, proj, 0, yb, state, ctx, 8.0, bf)), rows * W * 18)
        wg = torch.randn(10, 256, 256, device=dev).to(bf) * 0.05
        bg = torch.zeros(10, 256, device=dev)
        out[f"block_gates_{rows}"] = point(timed(lambda: ops.block_gates(u, wg, bg, wg, bg)), rows * W * 12 + 2 * wg.numel() * 2,
                                           2 * 2 * rows * W * 256)
        cw, cb = torch.randn(W, 4, device=dev), torch.zeros(W, device=dev)
        out[f"short_conv_{rows}"] = point(timed(lambda: ops.short_conv(proj, W, W, cw, cb, tail, ctx, activation=False, in_bias=cb)), rows * W * 8)
        # Mamba-2 beside it: 64 heads of 64, state 128, 8 groups (the sizes of movudra_sizes)
        heads, vdim, ns, groups = 64, 64, 128, 8
        xbc = torch.randn(rows, heads * vdim + 2 * groups * ns, device=dev)
        dt = torch.randn(rows, heads, device=dev)
        hv = torch.zeros(heads, device=dev)
        st2 = cache.unit_cache(1).state[1]
        out[f"mamba2_scan_{rows}"] = point(timed(lambda: ops.ssm_scan(xbc, dt, 0, hv, hv, hv, st2, ctx, heads, vdim, ns, groups)),
                                           rows * (xbc.shape[1] + heads * vdim) * 4 + (2 * B * st2[0].numel() * 4 if rows == B else 0))
    # attention: 16 heads of 128 over 4 key/value heads, window 1,024, blocks of 16
    H, G, dim, window, pool = 16, 4, 128, 1024, 16
    for label, n_new, B, prompt in (("prefill_2048", 2048, 1, 0), ("prefill_8192", 8192, 1, 0), ("decode_b8_at_4096", 1, 8, 4095),
                                    ("decode_b8_at_32768", 1, 8, 32767)):
        tokens, blocks = KVSpec(G, dim, window, value_dim=dim), KVSpec(G, dim, window, value_dim=dim, stride=pool)
        plain = KVSpec(2 * G, dim, 0)           # Qwen3's attention beside it: 8 key/value heads, every key visible
        n_ctx = prompt + n_new
        cache = CacheManager([((tokens, blocks), None, None), (plain, None, None)], B * n_ctx + 64 * B, B, n_ctx + 64, bf, dev)
        slots = cache.open(B)
        if prompt:
            build_step_context(cache, [StepEntry(s, [0] * prompt, []) for s in slots], 10, dev)
            for s in slots:
                cache.advance(s, prompt)
        for unit in (cache.unit_cache(0), cache.unit_cache(0).more[0], cache.unit_cache(1)):
            unit.k_pool.normal_()
            unit.v_pool.normal_()
        ctx = build_step_context(cache, [StepEntry(s, [0] * n_new, []) for s in slots], 10, dev)[0]
        rows = B * n_new
        u0, u1, u2 = cache.unit_cache(0), cache.unit_cache(0).more[0], cache.unit_cache(1)
        q = torch.randn(rows, H, dim, device=dev).to(bf)
        cs = torch.ones(rows, dim // 2, device=dev)
        t0, t1, t2 = (ctx.page_tables[u.group_id] for u in (u0, u1, u2))
        if n_new > 1:       # keys a query sees: up to `window` tokens and (position - window) / pool blocks; 4 FLOPs per key and value
            seen = sum(min(p + 1, window) + max(0, (p - window + 1) // pool) for p in range(n_new))
            full = n_new * (n_new + 1) // 2
            out[f"window_pool_attention_{label}"] = point(timed(lambda: ops.pool_attention(q, u0.k_pool, u0.v_pool, u1.k_pool, u1.v_pool, t0, t1, ctx, cs, cs, 0.09, window, pool, False), reps=3),
                                                          flops=4 * H * dim * seen)
            out[f"qwen3_attention_{label}"] = point(timed(lambda: ops.attn_prefill(q, u2.k_pool, u2.v_pool, t2, ctx.cu_seqlens, ctx.pos0, ctx.max_new, 0.09), reps=3),
                                                    flops=4 * H * dim * full)
        else:               # a decode step reads the visible keys and values of every key/value head once
            seen = min(n_ctx, window) + max(0, (n_ctx - window) // pool)
            out[f"window_pool_attention_{label}"] = point(timed(lambda: ops.pool_attention(q, u0.k_pool, u0.v_pool, u1.k_pool, u1.v_pool, t0, t1, ctx, cs, cs, 0.09, window, pool, False)),
                                                          B * G * seen * 2 * dim * 2)
            out[f"qwen3_attention_{label}"] = point(timed(lambda: ops.attn_decode(q, u2.k_pool, u2.v_pool, t2, ctx.seq_len, 0.09, ctx.max_len)),
                                                    B * 2 * G * n_ctx * 2 * dim * 2)
        del cache
        torch.cuda.empty_cache()
    return out


def punolix_kernels(torch, np, peaks) -> dict:
    """The Punolix design's own kernels alone at the sizes of ``punolix_sizes``, each beside the like kernel of a model the
    library had, with the bytes or FLOPs it must move and the share of the measured peak that this comes to: attention with
    two capped score maps and attention inside chunks, in prompts of 2,048 and 8,192 tokens and in decode steps (beside
    Qwen3's attention: its tcgen05 and ``mma.sync`` prompt kernels and its decode kernel), the preparation of q, k and v,
    and the gated linear recurrence (beside the gated delta rule's)."""
    from questwend_b200.cache.manager import CacheManager
    from questwend_b200.engine.engine import StepEntry, build_step_context
    from questwend_b200.kernels import ops
    from questwend_b200.parts.base import KVSpec, StateSpec
    dev, bf = torch.device("cuda:0"), torch.bfloat16
    hbm, tf = peaks["hbm_gbs"] * 1e9, peaks["bf16_tflops"] * 1e12
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)

    def timed(fn, reps=7):
        times = []
        for _ in range(reps + 3):
            flush.zero_()                                         # L2 holds nothing of the last run
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            fn()
            b.record()
            torch.cuda.synchronize()
            times.append(a.elapsed_time(b) * 1e3)
        return statistics.median(times[3:])

    def point(us, n_bytes=0, flops=0):
        p = {"us": round(us, 1)}
        if n_bytes:
            p.update(gb_s=round(n_bytes / us / 1e3, 1), hbm_frac=round(n_bytes / (us * 1e-6) / hbm, 3))
        if flops:
            p.update(tflops=round(flops / us / 1e6, 1), tensor_frac=round(flops / (us * 1e-6) / tf, 3))
        return p

    out = {}
    H, G, chunk, cap = 16, 4, 1024, 50.0
    for label, n_new, B, prompt in (("prefill_2048", 2048, 1, 0), ("prefill_8192", 8192, 1, 0), ("decode_b8_at_4096", 1, 8, 4095),
                                    ("decode_b8_at_32768", 1, 8, 32767)):
        two, one, plain = KVSpec(G, 2 * 64, 0, value_dim=128), KVSpec(G, 128, 0, value_dim=128), KVSpec(G, 128, 0)
        n_ctx = prompt + n_new
        cache = CacheManager([(two, None, None), (one, None, None), (plain, None, None)], B * n_ctx + 64 * B, B, n_ctx + 64, bf, dev)
        slots = cache.open(B)
        if prompt:
            build_step_context(cache, [StepEntry(s, [0] * prompt, []) for s in slots], 10, dev)
            for s in slots:
                cache.advance(s, prompt)
        units = [cache.unit_cache(i) for i in range(3)]
        for unit in units:
            unit.k_pool.normal_()
            unit.v_pool.normal_()
        ctx = build_step_context(cache, [StepEntry(s, [0] * n_new, []) for s in slots], 10, dev)[0]
        rows = B * n_new
        u0, u1, u2 = units
        t0, t1, t2 = (ctx.page_tables[u.group_id] for u in units)
        q2 = torch.randn(rows, H, 2 * 64, device=dev).to(bf)
        q1 = torch.randn(rows, H, 128, device=dev).to(bf)
        diff = lambda: ops.maps_attention(q2, u0.k_pool, u0.v_pool, t0, ctx, 2, 0.125, softcap=cap, lam=0.6, norm_out=True, eps=1e-5, out_scale=0.2)
        uncapped = lambda: ops.maps_attention(q2, u0.k_pool, u0.v_pool, t0, ctx, 2, 0.125, lam=0.6, norm_out=True, eps=1e-5, out_scale=0.2)
        chunked = lambda: ops.maps_attention(q1, u1.k_pool, u1.v_pool, t1, ctx, 1, 0.09, chunk=chunk)
        if n_new > 1:       # per (query, visible key): 2 FLOPs per key value and 2 per value, for every map
            full = n_new * (n_new + 1) // 2
            inside = sum(p % chunk + 1 for p in range(n_new))
            out[f"differential_attention_{label}"] = point(timed(diff, reps=3), flops=H * full * 2 * (2 * 64 + 2 * 128))
            out[f"differential_attention_no_cap_{label}"] = point(timed(uncapped, reps=3), flops=H * full * 2 * (2 * 64 + 2 * 128))
            out[f"chunked_attention_{label}"] = point(timed(chunked, reps=3), flops=H * inside * 4 * 128)
            for impl in ("tc", "mma"):
                out[f"qwen3_attention_{impl}_{label}"] = point(timed(lambda: ops.attn_prefill(q1, u2.k_pool, u2.v_pool, t2, ctx.cu_seqlens, ctx.pos0, ctx.max_new, 0.09, impl=impl), reps=3),
                                                               flops=H * full * 4 * 128)
                seen = sum(min(p + 1, chunk) for p in range(n_new))
                out[f"qwen3_attention_{impl}_window_{chunk}_{label}"] = point(timed(lambda: ops.attn_prefill(q1, u2.k_pool, u2.v_pool, t2, ctx.cu_seqlens, ctx.pos0, ctx.max_new, 0.09, window=chunk, impl=impl), reps=3),
                                                                              flops=H * seen * 4 * 128)
        else:               # a decode step reads the visible keys and values of every key/value head once
            inside = (n_ctx - 1) % chunk + 1
            out[f"differential_attention_{label}"] = point(timed(diff), B * G * n_ctx * (2 * 64 + 128) * 2)
            out[f"chunked_attention_{label}"] = point(timed(chunked), B * G * inside * (128 + 128) * 2)
            out[f"qwen3_attention_{label}"] = point(timed(lambda: ops.attn_decode(q1, u2.k_pool, u2.v_pool, t2, ctx.seq_len, 0.09, ctx.max_len)),
                                                    B * G * n_ctx * 2 * 128 * 2)
        # what stands in front of the scores: bias, norm of q and k, rotation, cache write (float in, bfloat16 out)
        n_cols = (H + G) * 128 + G * 128
        qkv = torch.randn(rows, n_cols, device=dev)
        bias, nw, cs = torch.zeros(n_cols, device=dev), torch.ones(128, device=dev), torch.ones(rows, 64, device=dev)
        out[f"maps_prep_{label}"] = point(timed(lambda: ops.maps_prep(qkv, bias, nw, nw, cs, cs, ctx, t1, u1.k_pool, u1.v_pool, H, G, 1, 128, 128, 128, False, 1e-5)),
                                          rows * n_cols * 6)
        del cache, units, u0, u1, u2
        torch.cuda.empty_cache()
    # the recurrences: one prompt of 2,048 tokens, and a step of 8 single tokens.  Gated linear attention: 4 heads of
    # 256 x 512; the gated delta rule beside it: 16 heads of 128 x 128 (the same 0.5 M numbers of state a sequence)
    for rows, B in ((2048, 1), (8, 8)):
        cache = CacheManager([(None, StateSpec((4, 512, 256)), None), (None, StateSpec((16, 128, 128)), None)], 4096, 8, 4096, bf, dev)
        slots = cache.open(B)
        ctx = build_step_context(cache, [StepEntry(s, [0] * (rows // B), []) for s in slots], 10, dev)[0]
        heads, K, P = 4, 256, 512
        qkv = torch.randn(rows, heads * (2 * K + P), device=dev) * 0.1
        a_raw, a_bias = torch.randn(rows, heads * K, device=dev), torch.zeros(heads * K, device=dev)
        st = cache.unit_cache(0).state
        moved = rows * heads * (3 * K + 2 * P) * 4 + (2 * B * st[0].numel() * 4 if rows == B else 0)
        out[f"gated_linear_attention_scan_{rows}"] = point(timed(lambda: ops.gla_scan(qkv, a_raw, a_bias, st, ctx, heads, K, P, K ** -0.5, 16.0)), moved)
        heads, K, P = 16, 128, 128
        qkv2 = torch.randn(rows, heads * (2 * K + P), device=dev) * 0.1
        b_raw, a_raw2 = torch.randn(rows, heads, device=dev), torch.randn(rows, heads * K, device=dev)
        dt_bias, a_log = torch.zeros(heads * K, device=dev), torch.zeros(heads, device=dev)
        st2 = cache.unit_cache(1).state
        moved = rows * heads * (3 * K + 2 * P) * 4 + (2 * B * st2[0].numel() * 4 if rows == B else 0)
        out[f"gated_delta_rule_scan_{rows}"] = point(timed(lambda: ops.delta_rule(qkv2, b_raw, 0, a_raw2, dt_bias, a_log, st2, ctx, heads, heads, K, P, 1e-6, K ** -0.5)), moved)
        o = torch.randn(rows, 4 * 512, device=dev)
        gate = torch.randn(rows, 4 * 512, device=dev)
        w = torch.ones(512, device=dev)
        out[f"gated_head_norm_{rows}"] = point(timed(lambda: ops.gated_part_norm(o, gate, 0, w, 4, 1e-5, gate_first=False, out_dtype=bf, gate_activation="silu")),
                                               rows * 4 * 512 * 10)
        del cache
        torch.cuda.empty_cache()
    return out


def sagupel_kernels(torch, np, peaks) -> dict:
    """The Sagupel design's own kernels alone at the sizes of ``sagupel_sizes``, each beside the like kernel of a model the
    library had, with the bytes or FLOPs it must move and the share of the measured peak that this comes to: attention over
    a window with a distance bias and a sink, and attention with capped scores and mixed heads, in prompts of 2,048 and
    8,192 tokens and in decode steps (beside Qwen3's attention and Punolix's capped attention with two score maps), the
    preparation of q and k, retention and the delta rule with a decay per head (beside the delta rule with a decay per
    channel), the norm after the sum (beside the norm in front of it) and the input convolution."""
    from questwend_b200.cache.manager import CacheManager
    from questwend_b200.engine.engine import StepEntry, build_step_context
    from questwend_b200.kernels import ops
    from questwend_b200.parts.base import KVSpec, StateSpec
    dev, bf = torch.device("cuda:0"), torch.bfloat16
    hbm, tf = peaks["hbm_gbs"] * 1e9, peaks["bf16_tflops"] * 1e12
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)

    def timed(fn, reps=7):
        times = []
        for _ in range(reps + 3):
            flush.zero_()                                         # L2 holds nothing of the last run
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            fn()
            b.record()
            torch.cuda.synchronize()
            times.append(a.elapsed_time(b) * 1e3)
        return statistics.median(times[3:])

    def point(us, n_bytes=0, flops=0):
        p = {"us": round(us, 1)}
        if n_bytes:
            p.update(gb_s=round(n_bytes / us / 1e3, 1), hbm_frac=round(n_bytes / (us * 1e-6) / hbm, 3))
        if flops:
            p.update(tflops=round(flops / us / 1e6, 1), tensor_frac=round(flops / (us * 1e-6) / tf, 3))
        return p

    out = {}
    H, G, window, cap = 16, 4, 1024, 25.0
    slopes = torch.tensor([2.0 ** (-8.0 * (h + 1) / H) for h in range(H)], device=dev)
    sinks, temp = torch.zeros(H, device=dev), torch.ones(H, device=dev)
    mix = (torch.eye(H, device=dev) + 0.1 * torch.randn(H, H, device=dev)).contiguous()
    for label, n_new, B, prompt in (("prefill_2048", 2048, 1, 0), ("prefill_8192", 8192, 1, 0), ("decode_b8_at_4096", 1, 8, 4095),
                                    ("decode_b8_at_32768", 1, 8, 32767)):
        spec, two = KVSpec(G, 128, 0, value_dim=128), KVSpec(G, 2 * 64, 0, value_dim=128)
        n_ctx = prompt + n_new
        cache = CacheManager([(spec, None, None), (two, None, None)], B * n_ctx + 64 * B, B, n_ctx + 64, bf, dev)
        slots = cache.open(B)
        if prompt:
            build_step_context(cache, [StepEntry(s, [0] * prompt, []) for s in slots], 10, dev)
            for s in slots:
                cache.advance(s, prompt)
        u1, u2 = cache.unit_cache(0), cache.unit_cache(1)
        for unit in (u1, u2):
            unit.k_pool.normal_()
            unit.v_pool.normal_()
        ctx = build_step_context(cache, [StepEntry(s, [0] * n_new, []) for s in slots], 10, dev)[0]
        rows = B * n_new
        t1, t2 = ctx.page_tables[u1.group_id], ctx.page_tables[u2.group_id]
        q1 = torch.randn(rows, H, 128, device=dev).to(bf)
        q2 = torch.randn(rows, H, 2 * 64, device=dev).to(bf)
        gate = torch.randn(rows, H, device=dev)
        windowed = lambda: ops.bias_attention(q1, u1.k_pool, u1.v_pool, t1, ctx, 0.09, slopes=slopes, window=window, sinks=sinks)
        mixed = lambda: ops.bias_attention(q1, u1.k_pool, u1.v_pool, t1, ctx, 0.09, head_scale=temp, softcap=cap, head_mix=mix, gate=gate)
        capped = lambda: ops.bias_attention(q1, u1.k_pool, u1.v_pool, t1, ctx, 0.09, head_scale=temp, softcap=cap)
        punolix = lambda: ops.maps_attention(q2, u2.k_pool, u2.v_pool, t2, ctx, 2, 0.125, softcap=50.0, lam=0.6, norm_out=True, eps=1e-5, out_scale=0.2)
        if n_new > 1:       # per (query, visible key): 2 FLOPs per key value and 2 per value; mixed heads: the values of all G heads
            full = n_new * (n_new + 1) // 2
            seen = sum(min(p + 1, window) for p in range(n_new))
            out[f"window_attention_{label}"] = point(timed(windowed, reps=3), flops=H * seen * 4 * 128)
            out[f"mixed_heads_attention_{label}"] = point(timed(mixed, reps=3), flops=H * full * 2 * 128 * (1 + G))
            out[f"capped_attention_no_mix_{label}"] = point(timed(capped, reps=3), flops=H * full * 4 * 128)
            out[f"punolix_two_capped_maps_{label}"] = point(timed(punolix, reps=3), flops=H * full * 2 * (2 * 64 + 2 * 128))
            for impl in ("tc", "mma"):
                out[f"qwen3_attention_{impl}_{label}"] = point(timed(lambda: ops.attn_prefill(q1, u1.k_pool, u1.v_pool, t1, ctx.cu_seqlens, ctx.pos0, ctx.max_new, 0.09, impl=impl), reps=3),
                                                               flops=H * full * 4 * 128)
                out[f"qwen3_attention_{impl}_window_{window}_{label}"] = point(timed(lambda: ops.attn_prefill(q1, u1.k_pool, u1.v_pool, t1, ctx.cu_seqlens, ctx.pos0, ctx.max_new, 0.09, window=window, impl=impl), reps=3),
                                                                               flops=H * seen * 4 * 128)
        else:               # a decode step reads the visible keys and values of every key/value head once
            inside = min(n_ctx, window)
            out[f"window_attention_{label}"] = point(timed(windowed), B * G * inside * 2 * 128 * 2)
            out[f"mixed_heads_attention_{label}"] = point(timed(mixed), B * G * n_ctx * 2 * 128 * 2)
            out[f"capped_attention_no_mix_{label}"] = point(timed(capped), B * G * n_ctx * 2 * 128 * 2)
            out[f"punolix_two_capped_maps_{label}"] = point(timed(punolix), B * G * n_ctx * (2 * 64 + 128) * 2)
            out[f"qwen3_attention_{label}"] = point(timed(lambda: ops.attn_decode(q1, u1.k_pool, u1.v_pool, t1, ctx.seq_len, 0.09, ctx.max_len)),
                                                    B * G * n_ctx * 2 * 128 * 2)
            out[f"qwen3_attention_window_{window}_{label}"] = point(timed(lambda: ops.attn_decode(q1, u1.k_pool, u1.v_pool, t1, ctx.seq_len, 0.09, ctx.max_len, window=window)),
                                                                    B * G * inside * 2 * 128 * 2)
        # what stands in front of the scores: norm of q and k, rotation, cache write (float in, bfloat16 out); the values are the keys
        n_cols = (H + G) * 128
        qk = torch.randn(rows, n_cols, device=dev)
        nw, cs = torch.ones(128, device=dev), torch.ones(rows, 64, device=dev)
        out[f"bias_prep_{label}"] = point(timed(lambda: ops.bias_prep(qk, None, nw, nw, cs, cs, ctx, t1, u1.k_pool, u1.v_pool, H, G, 128, 128, 128, False, 1e-5, values_are_keys=True)),
                                          rows * (n_cols * 4 + (H + 2 * G) * 128 * 2))
        qkv = torch.randn(rows, n_cols + G * 128, device=dev)
        out[f"punolix_maps_prep_{label}"] = point(timed(lambda: ops.maps_prep(qkv, None, nw, nw, cs, cs, ctx, t1, u1.k_pool, u1.v_pool, H, G, 1, 128, 128, 128, False, 1e-5)),
                                                  rows * (n_cols + G * 128) * 6)
        del cache, u1, u2
        torch.cuda.empty_cache()
    # the recurrences, 16 heads of 128 x 128: one prompt of 2,048 tokens, and a step of 8 single tokens
    for rows, B in ((2048, 1), (8, 8)):
        heads, K, P = 16, 128, 128
        cache = CacheManager([(None, StateSpec((heads, P, K)), None)], 4096, 8, 4096, bf, dev)
        slots = cache.open(B)
        ctx = build_step_context(cache, [StepEntry(s, [0] * (rows // B), []) for s in slots], 10, dev)[0]
        st = cache.unit_cache(0).state
        moved = rows * heads * (2 * K + 2 * P) * 4 + (2 * B * st[0].numel() * 4 if rows == B else 0)
        qkv = torch.randn(rows, heads * (2 * K + P), device=dev) * 0.1
        cs = torch.ones(rows, 64, device=dev)
        decay = torch.full((heads,), 0.98, device=dev)
        out[f"retention_scan_{rows}"] = point(timed(lambda: ops.retention_scan(qkv, cs, cs, 128, decay, st, ctx, heads, K, P, 1.0, K ** -0.5)), moved)
        proj = torch.randn(rows, 4 * K * 2 + heads * P + 2 * heads, device=dev) * 0.1
        qkv4 = torch.randn(rows, 4 * K * 2 + heads * P, device=dev) * 0.1
        C = 4 * K * 2 + heads * P
        dt_bias, a_log = torch.zeros(heads, device=dev), torch.zeros(heads, device=dev)
        out[f"delta_rule_decay_per_head_{rows}"] = point(timed(lambda: ops.delta_rule(qkv4, proj, C, proj, dt_bias, a_log, st, ctx, heads, 4, K, P, 1e-6, K ** -0.5, per_head=True, a_col0=C + heads)),
                                                         rows * (2 * 4 * K + heads * P * 2) * 4 + (2 * B * st[0].numel() * 4 if rows == B else 0))
        qkv2 = torch.randn(rows, heads * (2 * K + P), device=dev) * 0.1
        b_raw, a_raw2 = torch.randn(rows, heads, device=dev), torch.randn(rows, heads * K, device=dev)
        dt_bias2 = torch.zeros(heads * K, device=dev)
        out[f"delta_rule_decay_per_channel_{rows}"] = point(timed(lambda: ops.delta_rule(qkv2, b_raw, 0, a_raw2, dt_bias2, a_log, st, ctx, heads, heads, K, P, 1e-6, K ** -0.5)),
                                                            rows * heads * (3 * K + 2 * P) * 4 + (2 * B * st[0].numel() * 4 if rows == B else 0))
        # the stream's kernels at width 2,048
        D = 2048
        h, y, w = torch.randn(rows, D, device=dev), torch.randn(rows, D, device=dev), torch.ones(D, device=dev)
        out[f"norm_after_the_sum_{rows}"] = point(timed(lambda: ops.rmsnorm_mix(h, y, w, 1e-5, 2.0, bf)), rows * D * 14)
        out[f"norm_before_with_its_sum_{rows}"] = point(timed(lambda: ops.rmsnorm(h, w, 1e-5, bf, delta=y, write_sum=True)), rows * D * 14)
        tail = torch.zeros(8, 2, D, device=dev)
        cw = torch.randn(D, 3, device=dev)
        out[f"input_convolution_{rows}"] = point(timed(lambda: ops.short_conv(h, 0, D, cw, None, tail, ctx, activation=False, plus_input=True, out_dtype=bf)), rows * D * 6)
        del cache
        torch.cuda.empty_cache()
    return out


def reference_arm(args) -> int:
    """kishida/questwend itself, unmodified, through its own public classes (baseline/ref_bench.cpp), on the same sizes.
    Nothing of questwend_b200 is imported on this path."""
    def unavailable(why: str) -> int:
        print(json.dumps({"impl": "reference", "unavailable": why}))
        return 0
    exe = os.path.join(ROOT, "baseline", "_ref", "bin", "qw_ref_bench")
    if not os.path.exists(exe):
        return unavailable("the reference's CUDA build is not in baseline/_ref/bin (python baseline/build_reference.py "
                           "makes it from the CMake project; pip cannot install a project without setup.py or pyproject.toml)")
    if args.gpus != 1:
        return unavailable("kishida/questwend runs on one GPU")
    cfgd = MODELS[args.model]
    layers = args.layers or cfgd["num_hidden_layers"]
    need = 2 * (layers * (cfgd["hidden_size"] * (cfgd["num_attention_heads"] + 2 * cfgd["num_key_value_heads"]) * cfgd["head_dim"]
                          + cfgd["num_attention_heads"] * cfgd["head_dim"] * cfgd["hidden_size"]
                          + 3 * cfgd["hidden_size"] * cfgd["intermediate_size"])
                + 2 * cfgd["vocab_size"] * cfgd["hidden_size"]) + (1 << 30)
    place = None
    for cand in ("/dev/shm", tempfile.gettempdir()):
        try:
            if shutil.disk_usage(cand).free > need:
                place = cand
                break
        except OSError:
            pass
    if place is None:
        return unavailable(f"no room for a {need / 1e9:.0f} GB GGUF of random weights in /dev/shm or the temporary folder")
    warmup, steps = max(3, args.warmup), max(1, args.steps)
    peaks, peak_source = load_peaks()
    tmp = tempfile.mkdtemp(prefix="qw_ref_bench_", dir=place)
    gguf = os.path.join(tmp, "random.gguf")
    cmd = [exe, "--gguf", gguf, "--layers", str(layers), "--hidden", str(cfgd["hidden_size"]),
           "--heads", str(cfgd["num_attention_heads"]), "--kv-heads", str(cfgd["num_key_value_heads"]),
           "--head-dim", str(cfgd["head_dim"]), "--inter", str(cfgd["intermediate_size"]), "--vocab", str(cfgd["vocab_size"]),
           "--n-ctx", str(N_CTX), "--prompt", str(args.ref_prompt or PROMPT_LEN), "--prefill", str(PREFILL_TOKENS),
           "--sequences", str(args.batch), "--steps", str(steps), "--warmup", str(warmup)]
    clocks = ClockSampler()
    clocks.start()
    try:
        proc = subprocess.run(cmd, capture_output=True, text=True, timeout=1500)
    except subprocess.TimeoutExpired:
        clocks.stop()
        shutil.rmtree(tmp, ignore_errors=True)
        return unavailable("the reference's program did not finish within 1500 s")
    finally:
        shutil.rmtree(tmp, ignore_errors=True)
    clock_info = clocks.stop()
    sys.stderr.write(proc.stderr[-2000:])
    if proc.returncode != 0:
        last = (proc.stderr.strip().splitlines() or ["no message"])[-1]
        return unavailable(f"the reference's program ended with code {proc.returncode}: {last[:200]}")
    r = json.loads(proc.stdout.strip().splitlines()[-1])
    prompt = args.ref_prompt or PROMPT_LEN
    ctx = prompt + warmup + steps / 2.0
    wbytes = need - (1 << 30) - 2 * cfgd["vocab_size"] * cfgd["hidden_size"]          # the embedding table is only gathered from
    step_bytes = wbytes + ctx * kv_bytes_per_token(cfgd, layers)
    achieved = step_bytes * r["decode_tok_s"] / 1e9
    bucket = -(-int(ctx) // 32) * 32
    out = {"impl": "reference",
           "metric": "decode tokens/s (Qwen3-%s sizes, random bf16 weights, batch %d, n_ctx %d)" % (args.model.upper(), args.batch, N_CTX),
           "value": r["decode_tok_s"], "unit": "tokens/s", "n_gpus": 1, "steps": steps, "warmup": warmup,
           "ms_per_step": r["ms_per_token"], "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
           "data": "synthetic: seeded random weights in a GGUF written for the run, uniform random token ids",
           "config": {"model": f"qwen3-{args.model}-sizes", "layers": layers, "layers_full": cfgd["num_hidden_layers"],
                      "hidden_size": cfgd["hidden_size"], "heads": cfgd["num_attention_heads"],
                      "kv_heads": cfgd["num_key_value_heads"], "head_dim": cfgd["head_dim"],
                      "intermediate_size": cfgd["intermediate_size"], "vocab_size": cfgd["vocab_size"],
                      "global_batch": args.batch, "seq_len": N_CTX, "prompt_len": prompt,
                      "batching": "none in the reference: the sequences run one after the other, one token a step",
                      "parallelism": "single-gpu", "l2": "inputs_exceed_l2", "cuda_graph": "ggml's own", "peaks": peak_source,
                      "timing": "host clock around Runtime::decode, which returns after the logits are on the host"},
           "clocks": clock_info,
           "e2e": {"value": r["e2e_tok_s"], "unit": "tokens/s", "h2d_bytes_per_step": 4 + 4 + 8 + 2 * bucket,
                   "d2h_bytes_per_step": 4 * cfgd["vocab_size"]},
           "gpu_launches": None,
           "prefill": {"value": r["prefill_tok_s"], "tokens": r["prefill_tokens"], "ms": r["prefill_ms"],
                       "frac": (prefill_flops(cfgd, layers, r["prefill_tokens"]) / (r["prefill_ms"] / 1e3) /
                                (peaks["bf16_tflops"] * 1e12)) if r["prefill_ms"] else None},
           "roofline": {"bound": "hbm", "achieved": achieved, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                        "frac": achieved / peaks["hbm_gbs"], "of": peak_source},
           "points": {"decode_b1": r["decode_tok_s"]}}
    print(json.dumps(out))
    return 0


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=128)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--model", default="8b", choices=sorted(MODELS) + ["movudra", "roritar", "roritar-kernels", "punolix", "punolix-kernels", "sagupel", "sagupel-kernels"],
                    help="8b: the benchmark; 0.6b, 32b: its other workloads alone; movudra, roritar, punolix, sagupel: that design at real layer "
                         "sizes beside Qwen3 layers of the same width and depth; roritar-kernels, punolix-kernels, sagupel-kernels: its own kernels alone, each "
                         "beside the like kernel of a model the library had")
    ap.add_argument("--layers", type=int, default=0, help="fewer layers than the model has (named in config)")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--skip-points", action="store_true", help="leave out batch 1 / 64, the e2e run and the other models")
    ap.add_argument("--skip-other-models", action="store_true", help="leave out the 0.6B and 32B workloads")
    ap.add_argument("--ref-prompt", type=int, default=0, help="reference arm: another prompt length (a first, small call)")
    args = ap.parse_args()

    if args.impl == "reference":
        return reference_arm(args)
    if args.gpus != 1:
        print(f"bench.py: this library runs on one GPU; --gpus {args.gpus} is not supported")
        return 2
    warmup = max(3, args.warmup)
    steps = max(1, args.steps)
    if PROMPT_LEN + warmup + steps + 1 > N_CTX:
        print(f"bench.py: {PROMPT_LEN} prompt tokens + {warmup} + {steps} steps exceed the context of {N_CTX}")
        return 2

    import numpy as np
    import torch
    import questwend_b200 as qw

    peaks, peak_source = load_peaks()
    if args.model == "movudra":
        print(json.dumps({"metric": "Movudra at real layer sizes beside Qwen3 layers of equal width and depth", "n_gpus": 1,
                          "dtype": "bf16", "data": "synthetic: seeded random weights and uniform random token ids",
                          "peaks": peak_source, "points": movudra_workload(torch, np, peaks, steps, warmup)}))
        return 0
    if args.model == "roritar":
        designs = (("roritar", roritar_sizes()), ("qwen3_same_size", qwen3_beside()))
        print(json.dumps({"metric": "Roritar at real layer sizes beside Qwen3 layers of equal width and depth", "n_gpus": 1,
                          "dtype": "bf16", "data": "synthetic: seeded random weights and uniform random token ids",
                          "peaks": peak_source, "points": movudra_workload(torch, np, peaks, steps, warmup, designs)}))
        return 0
    if args.model == "roritar-kernels":
        print(json.dumps({"metric": "Roritar's kernels alone, each beside the like kernel of an earlier model", "n_gpus": 1,
                          "dtype": "bf16", "data": "synthetic: random tensors of the sizes of roritar_sizes; L2 flushed between runs",
                          "peaks": peak_source, "points": roritar_kernels(torch, np, peaks)}))
        return 0
    if args.model == "punolix":
        designs = (("punolix", punolix_sizes()), ("qwen3_same_size", qwen3_beside()))
        print(json.dumps({"metric": "Punolix at real layer sizes beside Qwen3 layers of equal width and depth", "n_gpus": 1,
                          "dtype": "bf16", "data": "synthetic: seeded random weights and uniform random token ids",
                          "peaks": peak_source, "points": movudra_workload(torch, np, peaks, steps, warmup, designs)}))
        return 0
    if args.model == "punolix-kernels":
        print(json.dumps({"metric": "Punolix's kernels alone, each beside the like kernel of an earlier model", "n_gpus": 1,
                          "dtype": "bf16", "data": "synthetic: random tensors of the sizes of punolix_sizes; L2 flushed between runs",
                          "peaks": peak_source, "points": punolix_kernels(torch, np, peaks)}))
        return 0
    if args.model == "sagupel":
        designs = (("sagupel", sagupel_sizes()), ("punolix_same_size", punolix_sizes()), ("qwen3_same_size", qwen3_beside()))
        print(json.dumps({"metric": "Sagupel at real layer sizes beside Punolix and Qwen3 layers of equal width and depth", "n_gpus": 1,
                          "dtype": "bf16", "data": "synthetic: seeded random weights and uniform random token ids",
                          "peaks": peak_source, "points": movudra_workload(torch, np, peaks, steps, warmup, designs)}))
        return 0
    if args.model == "sagupel-kernels":
        print(json.dumps({"metric": "Sagupel's kernels alone, each beside the like kernel of an earlier model", "n_gpus": 1,
                          "dtype": "bf16", "data": "synthetic: random tensors of the sizes of sagupel_sizes; L2 flushed between runs",
                          "peaks": peak_source, "points": sagupel_kernels(torch, np, peaks)}))
        return 0
    if args.model != "8b":                      # one of the other workloads alone, as a line of its own
        points = small_model_workload(torch, np, peaks) if args.model == "0.6b" else large_model_workload(torch, np, peaks)
        print(json.dumps({"metric": f"Qwen3-{args.model.upper()} sizes workload", "n_gpus": 1, "dtype": "bf16",
                          "data": "synthetic: seeded random weights and uniform random token ids", "peaks": peak_source,
                          "points": points}))
        return 0
    layers = args.layers or QWEN3_8B["num_hidden_layers"]
    max_batch = max(args.batch, 1 if args.skip_points else 64)
    engine, cfgd = make_engine(QWEN3_8B, layers, max_batch, max(PROMPT_LEN + 512, -(-(PREFILL_TOKENS + 64) // max_batch)))
    rng = np.random.default_rng(0)
    wbytes = weight_bytes(engine)
    kv_tok = kv_bytes_per_token(cfgd, layers)

    # ---- the headline: decode at the given batch, device-timed
    clocks = ClockSampler()
    clocks.start()
    main_run = decode_run(engine, torch, args.batch, warmup, steps, rng)
    clock_info = clocks.stop()
    step_s = main_run["ms_per_step"] / 1e3
    step_bytes = wbytes + args.batch * main_run["mean_ctx"] * kv_tok
    achieved = step_bytes / step_s / 1e9

    # ---- prefill of one 2,048-token prompt
    pf_ms = time_prefill(engine, torch, rng, PREFILL_TOKENS)
    pf_flops = prefill_flops(cfgd, layers, PREFILL_TOKENS)
    prefill = {"value": PREFILL_TOKENS / (pf_ms / 1e3), "tokens": PREFILL_TOKENS, "ms": pf_ms,
               "frac": pf_flops / (pf_ms / 1e3) / (peaks["bf16_tflops"] * 1e12)}

    # ---- other batch sizes, and the same batch through the Python entry point
    points, e2e = {}, None
    if not args.skip_points:
        for b in (1, 64):
            r = decode_run(engine, torch, b, 3, 32, rng)
            points[f"decode_b{b}"] = r["tok_s"]
            points[f"decode_b{b}_frac"] = (wbytes + b * r["mean_ctx"] * kv_tok) / (r["ms_per_step"] / 1e3) / 1e9 / peaks["hbm_gbs"]
        prompts = [rng.integers(0, engine.vocab_size, PROMPT_LEN).tolist() for _ in range(args.batch)]
        stats = qw.GenerationStats()
        qw.generate(engine, prompts, max_new_tokens=warmup + 1, ignore_eos=True)          # warm the graphs
        # one call: the prompts, `warmup` untimed decode steps, then the `steps` timed ones (the loop's own clock around
        # each step: tokens from pinned host memory in, the step, its ids back on the host)
        qw.generate(engine, prompts, max_new_tokens=warmup + steps + 1, ignore_eos=True, stats=stats)
        timed = stats.step_seconds[-steps:]
        e2e = {"value": args.batch * len(timed) / sum(timed), "unit": "tokens/s",
               "h2d_bytes_per_step": 4 * args.batch, "d2h_bytes_per_step": 4 * args.batch,
               "steps": len(timed), "warmup_steps": len(stats.step_seconds) - len(timed),
               "value_all_steps": args.batch * stats.steps / stats.decode_seconds}
        for n in (4096,):          # the whole context of the benchmark's configuration
            ms = time_prefill(engine, torch, rng, n, reps=3)
            points[f"prefill_{n}"] = n / (ms / 1e3)
            points[f"prefill_{n}_frac"] = prefill_flops(cfgd, layers, n) / (ms / 1e3) / (peaks["bf16_tflops"] * 1e12)
    release(engine, torch)
    del engine
    if not (args.skip_points or args.skip_other_models):
        points.update(small_model_workload(torch, np, peaks))
        points.update(large_model_workload(torch, np, peaks))

    out = {
        "metric": "decode tokens/s (Qwen3-8B sizes, random bf16 weights, batch %d, n_ctx %d)" % (args.batch, N_CTX),
        "value": main_run["tok_s"], "unit": "tokens/s", "n_gpus": 1, "steps": steps, "warmup": warmup,
        "ms_per_step": main_run["ms_per_step"], "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic: seeded random weights and uniform random token ids",
        "config": {"model": "qwen3-8b-sizes", "layers": layers, "layers_full": QWEN3_8B["num_hidden_layers"],
                   "hidden_size": cfgd["hidden_size"], "heads": cfgd["num_attention_heads"],
                   "kv_heads": cfgd["num_key_value_heads"], "head_dim": cfgd["head_dim"],
                   "intermediate_size": cfgd["intermediate_size"], "vocab_size": cfgd["vocab_size"],
                   "global_batch": args.batch, "seq_len": N_CTX, "prompt_len": PROMPT_LEN,
                   "mean_ctx_timed": main_run["mean_ctx"], "parallelism": "single-gpu",
                   "l2": "inputs_exceed_l2", "cuda_graph": True, "peaks": peak_source},
        "clocks": clock_info, "e2e": e2e, "gpu_launches": main_run["launches_per_step"] * steps,
        "prefill": prefill,
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                     "frac": achieved / peaks["hbm_gbs"], "of": peak_source},
        "points": points,
    }
    print(json.dumps(out))
    return 0


if __name__ == "__main__":
    sys.exit(main())
