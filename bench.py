#!/usr/bin/env python3
"""Decode and prefill throughput of the engine at the Qwen2.5 layer sizes, random weights.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--batch 8] [--context 2048] [--layers L]
                    [--shape qwen2.5-0.5b | --model DIR] [--dtype bf16|f32] [--only headline,fp32,...]

Prints ONE JSON line.  A step is one decode step of `batch` requests that each hold
`context` tokens: the model, the sampler and the copy of the sampled tokens to pinned host
memory.  `value` is decoded tokens per second timed on the device with CUDA events around
K such steps after W warm-up steps (the next step's tokens are taken from the sampler's
output on the device); the block of K steps is timed three times and the median block is
reported, with the spread beside it.  `logits_only` is the same without sampler and copy.
`e2e` is the same through the Python entry point (`Engine.step`: host token ids in
through pinned memory, sampled token ids read by the host, every step).  `prefill` is one
request of 2,048 tokens in one step.  `roofline` relates the bytes a decode step has to
read (every weight once, and the cache of the live requests) to the measured copy
bandwidth.  Every step reads about a gigabyte of weights, far more than the 126 MB of L2,
so nothing needs flushing between steps.

Beside the headline the default run measures, under keys of their own:

* `fp32`: the true 32-bit path at the same sizes (decode at the headline batch, prefill);
* `serving_1p5b`: Qwen2.5-1.5B sizes, 64 requests with prompts of 128 to 2,048 tokens and
  256 new tokens each, through `Engine` with continuous batching (generated and prompt
  tokens per second, time to first token, preemptions);
* `mixed_7b`: Qwen2.5-7B sizes, one step of eight 512-row portions of 4,096-token prompts
  (3,584 earlier tokens in the cache) beside 56 decoding rows at 1,024-token contexts.

`--only venarax` (not part of the default run) times the Venarax design (parallel layers, attention with a sink,
latent attention, clamped gated feed-forward) at the layer sizes of the three Qwen2.5 shapes beside the dense decoder
at the same sizes: decode at `--batch` and `--context`, one prompt of `--prefill` tokens, and the design's kernels
alone beside the like kernels of the dense decoder, each with its fraction of the measured peak.

`--only fozutar` (not part of the default run either) does the same for the Fozutar design (attention in chunks with a
soft cap and a bias by distance, gated linear attention, dense and routed feed-forwards).

`--only modadra` (not part of the default run either) times the Modadra design (windowed attention with a partial rotation,
one more in the softmax's denominator and head gates beside a gated delta rule, their normed outputs averaged; experts
without a gate behind a router of sigmoid scores with groups) beside the Fozutar design and the dense decoder at the same
sizes, and its kernels alone beside the like kernels of those.

`--only varolix` (not part of the default run either) times the Varolix design (rotary attention with biases and stretched
waves; normed attention with a query temperature beside a matrix memory with exponential gates, summed with weights; latent
attention with a query latent, a sink and head gates; dense gated feed-forwards) beside the Fozutar design (the closest one:
attention layers and layers with a matrix state, dense feed-forwards among its layers) and the dense decoder at the same
sizes, and its kernels alone beside the like kernels of those.

This engine runs on one GPU: for --gpus > 1 it says so and exits with 2.

    python bench.py --kernel attention_prefill

times the prompt attention kernel alone (2,048, 4,096 and 8,192 tokens) and prints a line of its own;
`--kernel gemm [--shape ...] [--prefill ROWS]` the four products of a layer with their fused epilogues beside the
library's.  `--profile decode|prefill|mixed` brackets that timed region with cudaProfilerStart/Stop, for a profiler
started with --profile-from-start off (the commands are in profiles/).
"""
from __future__ import annotations

import argparse
import gc
import json
import os
import statistics
import subprocess
import sys
import threading
import time

REPO = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, REPO)

_COMMON = {
    "architectures": ["Qwen2ForCausalLM"], "model_type": "qwen2", "rms_norm_eps": 1e-6, "rope_theta": 1000000.0,
    "max_position_embeddings": 32768, "use_sliding_window": False, "hidden_act": "silu", "torch_dtype": "bfloat16",
}
SHAPES = {
    "qwen2.5-0.5b": dict(_COMMON, vocab_size=151936, hidden_size=896, num_hidden_layers=24, num_attention_heads=14,
                         num_key_value_heads=2, intermediate_size=4864, tie_word_embeddings=True),
    "qwen2.5-1.5b": dict(_COMMON, vocab_size=151936, hidden_size=1536, num_hidden_layers=28, num_attention_heads=12,
                         num_key_value_heads=2, intermediate_size=8960, tie_word_embeddings=True),
    "qwen2.5-7b": dict(_COMMON, vocab_size=152064, hidden_size=3584, num_hidden_layers=28, num_attention_heads=28,
                       num_key_value_heads=4, intermediate_size=18944, tie_word_embeddings=False),
}
QWEN25_05B = SHAPES["qwen2.5-0.5b"]
# the reference's own figure for decode at batch 8 (RX 7900 XTX, float32 weights, short context)
PUBLISHED_DECODE_B8 = 626.0
PAGE = 64


def peaks():
    path = os.path.join(REPO, "MEASURED_PEAKS.json")
    if os.path.isfile(path):
        p = json.load(open(path))
        return {"hbm_gbs": p["hbm_gbs"], "bf16_tflops": p["bf16_tflops"], "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}


class ClockSampler(threading.Thread):
    """Samples SM clock and throttle reasons with nvidia-smi while the timed region runs."""

    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self):
        super().__init__(daemon=True)
        self.samples, self.stop_flag, self.proc = [], False, None

    def run(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", "0", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "100"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            for line in self.proc.stdout:
                if self.stop_flag:
                    break
                self.samples.append([x.strip() for x in line.split(",")])
        except OSError:
            pass

    def stop(self):
        self.stop_flag = True
        if self.proc is not None:
            self.proc.terminate()
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": []}
        rows = [s for s in self.samples if len(s) == 6 and s[0].isdigit()]
        if rows:
            out["sm_mhz"] = statistics.median(int(r[0]) for r in rows)
            out["sm_max_mhz"] = int(rows[0][1])
            names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
            out["reasons"] = [n for i, n in enumerate(names) if any(r[2 + i] == "Active" for r in rows)]
        return out


# ----------------------------------------------------------------- what a step has to read and to compute


def sizes(raw):
    d, i, v = raw["hidden_size"], raw["intermediate_size"], raw["vocab_size"]
    hq, hkv = raw["num_attention_heads"], raw["num_key_value_heads"]
    return d, i, v, hq, hkv, raw.get("head_dim", d // hq)


def weight_bytes(raw, layers, elt=2):
    """Every weight a step reads once: the layers, the final norm and the head (a tied table is read by the head)."""
    d, i, v, hq, hkv, hd = sizes(raw)
    per_layer = d * (hq + 2 * hkv) * hd + (hq + 2 * hkv) * hd + hq * hd * d + 3 * d * i + 2 * d
    return elt * (layers * per_layer + v * d + d)


def kv_bytes_per_token(raw, layers, elt=2):
    _, _, _, _, hkv, hd = sizes(raw)
    return elt * layers * 2 * hkv * hd


def decode_bytes(raw, layers, batch, context, elt=2):
    """Bytes one decode step has to read: every weight once, and the cache of the live requests."""
    return weight_bytes(raw, layers, elt) + kv_bytes_per_token(raw, layers, elt) * context * batch


def step_flops(raw, layers, rows, attended_keys, head_rows):
    """Multiply-adds x 2 of a step: `rows` token rows through the layers' matrices, `attended_keys` (query, key)
    pairs through the attention of every head, `head_rows` rows through the vocabulary head."""
    d, i, v, hq, hkv, hd = sizes(raw)
    matmul = 2 * rows * layers * (d * (hq + 2 * hkv) * hd + hq * hd * d + 3 * d * i)
    return matmul + 2 * 2 * attended_keys * hd * hq * layers + 2 * head_rows * v * d


def prefill_flops(raw, layers, tokens):
    return step_flops(raw, layers, tokens, tokens * (tokens + 1) // 2, 1)


def config_block(raw, layers, **more):
    d, i, v, hq, hkv, hd = sizes(raw)
    return {"layers": layers, "layers_of_configuration": raw["num_hidden_layers"], "hidden_size": d, "heads": hq,
            "kv_heads": hkv, "head_dim": hd, "intermediate_size": i, "vocab_size": v,
            "tied_embeddings": bool(raw["tie_word_embeddings"]), "page_size": PAGE, **more}


def free_device_memory():
    """After the caller has dropped its runner: gives the device memory back before the next workload is built."""
    import torch

    gc.collect()
    torch.cuda.empty_cache()


# ------------------------------------------------------------------------------------- one kernel alone


def time_gemm_pair_tc(torch, ops, a, pk) -> int:
    """The four products of a layer at `--prefill` rows: the repository's tcgen05 product with its fused epilogues (a
    pair of SMs per tile; the engine uses its gated form for the feed-forward from 1,024 rows on and the library for
    the other products above 16 rows) beside the library's."""
    raw = SHAPES[a.shape]
    h, inter = raw["hidden_size"], raw["intermediate_size"]
    hd = raw.get("head_dim", h // raw["num_attention_heads"])
    qkv = (raw["num_attention_heads"] + 2 * raw["num_key_value_heads"]) * hd
    m, dev = a.prefill, "cuda:0"
    g = torch.Generator(device=dev).manual_seed(0)
    rnd = lambda *shape, s=0.05: (torch.randn(*shape, device=dev, generator=g) * s).to(torch.bfloat16)
    x, xi = rnd(m, h, s=0.5), rnd(m, inter, s=0.5)
    w_qkv, w_o, w_gu, w_d = rnd(qkv, h), rnd(h, h), rnd(2 * inter, h), rnd(h, inter, s=0.02)
    res = torch.randn(m, h, device=dev, generator=g)
    nb = ops.gemm_pair_tc_stats_blocks(m, h)
    stats, copy = torch.ones(m, nb, device=dev), torch.empty(m, h, dtype=torch.bfloat16, device=dev)
    o_qkv, o_h = torch.empty(m, qkv, dtype=torch.bfloat16, device=dev), torch.empty(m, h, dtype=torch.bfloat16, device=dev)
    o_gu, o_i = torch.empty(m, 2 * inter, dtype=torch.bfloat16, device=dev), torch.empty(m, inter, dtype=torch.bfloat16, device=dev)

    def us(fn, reps=20):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            for _ in range(reps):
                fn()
        graph.replay()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        graph.replay()
        graph.replay()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / (2 * reps) * 1000

    if a.profile:  # one launch each of the gated product, the same product plain and the library's, for a profiler
        for _ in range(3):
            ops.gemm_pair_tc_silu_mul(x, w_gu, o_i)
            ops.gemm_pair_tc(x, w_gu, o_gu)
            torch.mm(x, w_gu.T, out=o_gu)
        torch.cuda.synchronize()
        torch.cuda.profiler.start()
        ops.gemm_pair_tc_silu_mul(x, w_gu, o_i)
        ops.gemm_pair_tc(x, w_gu, o_gu)
        torch.mm(x, w_gu.T, out=o_gu)
        torch.cuda.synchronize()
        torch.cuda.profiler.stop()
        assert ops.gemm_tc_status() == 0
        print(json.dumps({"kernel": "gemm_pair_tc", "shape": a.shape, "rows": m, "profiled": ["gate_up_silu_mul", "gate_up_plain", "library"]}))
        return 0
    out = {}
    for name, own, lib, flops in (
        ("qkv_norm_folded", lambda: ops.gemm_pair_tc(x, w_qkv, o_qkv, stats, nb, 1e-6), lambda: torch.mm(x, w_qkv.T, out=o_qkv), 2 * m * h * qkv),
        ("o_residual_add", lambda: ops.gemm_pair_tc_resadd(x, w_o, res, stats, copy), lambda: torch.mm(x, w_o.T, out=o_h), 2 * m * h * h),
        ("gate_up_silu_mul", lambda: ops.gemm_pair_tc_silu_mul(x, w_gu, o_i, stats, nb, 1e-6), lambda: torch.mm(x, w_gu.T, out=o_gu), 4 * m * h * inter),
        ("down_residual_add", lambda: ops.gemm_pair_tc_resadd(xi, w_d, res, stats, copy), lambda: torch.mm(xi, w_d.T, out=o_h), 2 * m * h * inter)):
        t_own, t_lib = us(own), us(lib)
        out[name] = {"own_us": round(t_own, 1), "own_tflops": round(flops / t_own / 1e6), "library_us": round(t_lib, 1),
                     "library_tflops": round(flops / t_lib / 1e6)}
    assert ops.gemm_tc_status() == 0
    print(json.dumps({"kernel": "gemm_pair_tc", "shape": a.shape, "rows": m, "dtype": "bf16", "products": out,
                      "note": "own: with the epilogue named; library: the plain product alone", "peaks": pk["source"]}))
    return 0


def time_attention_prefill(torch, ops, a, pk) -> int:
    """The prompt attention kernel alone: one sequence of 2,048, 4,096 and 8,192 tokens attending to itself through
    the paged cache, replayed as a CUDA graph of ten launches; CUDA events around the replays."""
    raw = SHAPES[a.shape]
    _, _, _, hq, hkv, hd = sizes(raw)
    page = PAGE
    dev, res = "cuda:0", {}
    for n in (512, 2048, 4096, 8192):
        torch.manual_seed(n)
        pages = n // page + 1
        kp = torch.randn((pages, hkv, page, hd), device=dev).to(torch.bfloat16)
        vp = torch.randn_like(kp)
        table = torch.arange(pages, dtype=torch.int32, device=dev).view(1, -1).contiguous()
        q = torch.randn((n, hq * hd), device=dev).to(torch.bfloat16)
        out = torch.empty_like(q)
        pos = torch.arange(n, dtype=torch.int32, device=dev)
        slot = torch.zeros(n, dtype=torch.int32, device=dev)
        t0 = torch.arange(0, n, 128, dtype=torch.int32, device=dev)
        tn = torch.full_like(t0, 128)
        tiles = t0.numel()
        splits, alone, run_tiles = ops.attention_prefill_tc_plan(tiles, hq, hkv, hd, n, tiles * (tiles + 1) // 2)  # the engine's own choice
        words = ops.attention_prefill_tc_scratch_words(t0.numel(), hq, hd, splits)
        scratch = torch.zeros(words, dtype=torch.float32, device=dev) if words else None
        counters = torch.zeros(t0.numel() * hq, dtype=torch.int32, device=dev) if words else None
        def run():
            ops.attention_prefill_tc(q, kp, vp, out, t0, tn, t0.numel(), pos, slot, table, hq, hkv, hd, None, hd ** -0.5,
                                     splits, scratch, counters, alone=alone, run_tiles=run_tiles)
        for _ in range(max(a.warmup, 3)):
            run()
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            for _ in range(10):
                run()
        g.replay()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        reps = max(1, a.steps // 10)
        e0.record()
        for _ in range(reps):
            g.replay()
        e1.record()
        torch.cuda.synchronize()
        us = e0.elapsed_time(e1) / (10 * reps) * 1000
        flops = 4 * hq * hd * n * (n + 1) / 2
        res[str(n)] = {"us": round(us, 1), "tflops": round(flops / us / 1e6, 1), "frac": round(flops / us / 1e6 / pk["bf16_tflops"], 3),
                       "key_splits": splits, "key_tiles_a_run": run_tiles, "heads_per_block": 1 if alone or hd == 64 else 2}
    assert ops.gemm_tc_status() == 0
    print(json.dumps({"kernel": "attention_prefill_tc", "heads": hq, "kv_heads": hkv, "head_dim": hd, "page_size": page,
                      "dtype": "bf16", "tokens": res, "peaks": pk["source"]}))
    return 0


# --------------------------------------------------------------------------- decode and prefill of one model


class DecodeBench:
    """A runner of one shape with helpers that fill contexts and time decode steps and a prefill."""

    def __init__(self, a, raw, layers, dtype, max_batch, max_seq, load_dir=None, config=None, vocab=None):
        import numpy as np
        import torch

        from machserve_b200 import ModelRunner
        from machserve_b200.config import config_from_json
        from machserve_b200.sampling.sampler import Sampler

        self.a, self.raw, self.layers, self.dtype = a, raw, layers, dtype
        self.torch, self.np = torch, np
        pages = max_batch * (-(-max_seq // PAGE)) + 8
        kw = dict(dtype=dtype, page_size=PAGE, num_pages=pages, max_requests=max_batch,
                  max_step_tokens=2048 + max_batch, max_seq_len=max_seq)
        if load_dir:
            self.runner = ModelRunner.from_model_dir(load_dir, **kw)
        elif config is not None:  # a configuration of any architecture, as its config.json would give it
            self.runner = ModelRunner.from_random(config_from_json(config), seed=0, on_device=True, **kw)
        else:
            cfg = dict(raw)
            cfg["num_hidden_layers"] = layers
            self.runner = ModelRunner.from_random(config_from_json(cfg), seed=0, on_device=True, **kw)
        self.sampler = Sampler(max_batch, self.runner.device)
        self.rng = np.random.default_rng(0)
        self.vocab = vocab or raw["vocab_size"]

    def release_all(self):
        for r in list(self.runner.cache.requests):
            self.runner.release(r)

    def fill(self, batch, context):
        from machserve_b200 import StepEntry

        self.release_all()
        for r in range(batch):
            toks = self.rng.integers(0, self.vocab, size=context)
            for at in range(0, context, 2048):
                self.runner.step([StepEntry(r, toks[at : at + 2048].tolist(), [])])
        self.torch.cuda.synchronize()

    def time_decode(self, batch, context, steps, warmup, blocks=3, sampled=True, profile=False):
        """ms per step of `blocks` blocks of `steps` decode steps (sorted), and the launches of one block.
        With `sampled`, a step is the model, the sampler and the copy of the tokens to pinned host memory, and the
        next step takes its tokens from the sampler's output on the device; without, the model alone."""
        from machserve_b200 import SamplingParams, StepEntry, ops

        torch, runner, sampler = self.torch, self.runner, self.sampler
        self.fill(batch, context)
        greedy, states = [SamplingParams()] * batch, [1] * batch
        toks = self.rng.integers(0, self.vocab, size=batch)
        first = [True]

        def one():
            if not sampled:
                runner.step([StepEntry(r, [int(toks[r])], [0]) for r in range(batch)])
                return
            if first[0]:
                entries = [StepEntry(r, [int(toks[r])], [0]) for r in range(batch)]
                first[0] = False
            else:
                entries = [StepEntry(r, [0], [0], from_sampled=r) for r in range(batch)]
            logits = runner.step(entries, sampled=sampler.tokens_on_device)
            sampler.launch(logits, greedy, states)

        for _ in range(warmup):
            one()
        torch.cuda.synchronize()
        times, launches = [], 0
        for b in range(blocks):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            l0 = ops.launches()
            if profile and b == 0:
                torch.cuda.profiler.start()  # a profiler started with --profile-from-start off sees these steps only
            e0.record()
            for _ in range(steps):
                one()
            e1.record()
            torch.cuda.synchronize()
            if profile and b == 0:
                torch.cuda.profiler.stop()
            times.append(e0.elapsed_time(e1) / steps)
            launches = ops.launches() - l0
        return sorted(times), launches

    def time_prefill(self, tokens, warmup, reps=5, profile=False):
        """Median ms of one request of `tokens` tokens in one step, logits at its last token, sampled."""
        from machserve_b200 import SamplingParams, StepEntry

        torch, runner = self.torch, self.runner
        self.release_all()
        times = []
        for it in range(warmup + reps):
            toks = self.rng.integers(0, self.vocab, size=tokens).tolist()
            torch.cuda.synchronize()
            last = it == warmup + reps - 1
            if profile and last:
                torch.cuda.profiler.start()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            logits = runner.step([StepEntry("p", toks, [tokens - 1])])
            self.sampler.launch(logits, [SamplingParams()], [1])
            e1.record()
            torch.cuda.synchronize()
            if profile and last:
                torch.cuda.profiler.stop()
            runner.release("p")
            if it >= warmup:
                times.append(e0.elapsed_time(e1))
        return statistics.median(times)

    def time_e2e(self, batch, context, steps, warmup):
        """Tokens per second through `Engine.step`: host ids in, sampled ids read by the host, every step."""
        from machserve_b200 import Engine, SamplingParams

        torch, runner = self.torch, self.runner
        self.release_all()
        eng = Engine(runner=runner, prefill_rows=2048)
        # (a request decodes while the prompts behind it are still read, one prompt a step: none may finish before the end)
        for _ in range(batch):
            eng.add(self.rng.integers(0, self.vocab, size=context).tolist(), steps + warmup + batch + 8, params=SamplingParams())
        while any(s.computed < len(s.prompt) for s in eng.scheduler.running) or eng.scheduler.waiting:
            eng.step()
        for _ in range(warmup):
            eng.step()
        torch.cuda.synchronize()
        h2d0, d2h0 = runner.h2d_bytes + eng.sampler.h2d_bytes, eng.sampler.d2h_bytes
        t0 = time.perf_counter()
        made = 0
        for _ in range(steps):
            made += len(eng.step())
        torch.cuda.synchronize()
        dt = time.perf_counter() - t0
        # counted from the tensors that were copied: the step's index arrays (token ids among them) and changed
        # block-table rows from pinned memory to the device; the sampled tokens and log-probabilities back
        out = {"value": round(made / dt, 1), "unit": "tokens/s",
               "h2d_bytes_per_step": round((runner.h2d_bytes + eng.sampler.h2d_bytes - h2d0) / steps, 1),
               "d2h_bytes_per_step": round((eng.sampler.d2h_bytes - d2h0) / steps, 1)}
        while not eng.all_done():
            eng.step()
        return out


# ------------------------------------------------------------------------------------ the other workloads


def workload_fp32(a, pk, raw, layers):
    """The true 32-bit path at the headline's sizes: decode at the headline batch and a prefill of 2,048 tokens."""
    steps = max(10, a.steps // 2)
    b = DecodeBench(a, raw, layers, "f32", a.batch, a.context + 4 * (steps + a.warmup) + a.batch + 64)
    times, launches = b.time_decode(a.batch, a.context, steps, a.warmup)
    ms = times[len(times) // 2]
    nbytes = decode_bytes(raw, layers, a.batch, a.context + a.warmup + steps * 3 // 2, elt=4)
    pms = b.time_prefill(2048, 1, reps=3)
    out = {"dtype": "fp32", "global_batch": a.batch, "seq_len": a.context, "steps": steps,
           "decode_tokens_per_s": round(a.batch * 1000.0 / ms, 1), "ms_per_step": round(ms, 4),
           "ms_min": round(times[0], 4), "ms_max": round(times[-1], 4), "gpu_launches_per_step": launches // steps,
           "hbm_gbs": round(nbytes / ms / 1e6, 1), "hbm_frac": round(nbytes / ms / 1e6 / pk["hbm_gbs"], 4),
           "prefill_tokens": 2048, "prefill_ms": round(pms, 3), "prefill_tokens_per_s": round(2048e3 / pms, 1),
           "prefill_tflops": round(prefill_flops(raw, layers, 2048) / pms / 1e9, 2),
           "matrix_products": "float32 multiply-adds on the CUDA cores, no reduced-precision mode"}
    b.release_all()
    del b
    free_device_memory()
    return out


def venarax_config(raw, layers, window=1024):
    """A Venarax configuration with the layer sizes of the Qwen2 shape `raw`: the same width, heads, key heads, head
    size, feed-forward size and vocabulary; every third layer a latent-attention layer (latent of four head sizes, half
    a head size of rotated coordinates, a window of `window` tokens), the others attention layers; no loop."""
    d, i, v, hq, hkv, hd = sizes(raw)
    att = {"type": "attention", "mixer": {"heads": hq, "kv_heads": hkv, "dim": hd, "vdim": hd, "scale": hd ** -0.5,
                                          "q_temp": {"coef": 0.1, "every": 1024}}, "mlp": {"kind": "dense", "ff": i, "limit": 7.0}}
    lat = {"type": "latent_attention", "mixer": {"heads": hq, "dim": hd, "rot_dim": hd // 2, "vdim": hd, "kv_rank": 4 * hd,
                                                 "scale": (hd + hd // 2) ** -0.5, "rot": {"base": 10000.0, "dims": hd // 2},
                                                 "mask": {"size": window}}, "mlp": {"kind": "dense", "ff": i, "limit": 7.0}}
    return {"architecture": "Venarax", "vocab": v, "width": d, "norm": {"eps": 1e-6},
            "layers": [lat if n % 3 == 2 else att for n in range(layers)]}


def time_venarax_kernels(torch, ops, raw, pk):
    """The new design's kernels alone, each beside the like kernel of the dense decoder at equal sizes (inputs larger
    than the L2; a CUDA graph of a few launches between events)."""
    d, inter, _, hq, hkv, hd = sizes(raw)
    dev, bf = "cuda:0", torch.bfloat16
    g = torch.Generator(device=dev).manual_seed(0)
    rnd = lambda *shape, dt=torch.float32: torch.randn(*shape, device=dev, generator=g).to(dt)

    def us(fn, reps=5):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            for _ in range(reps):
                fn()
        graph.replay()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        graph.replay()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / reps * 1000

    out = {}

    def entry(name, t_new, t_like, nbytes=None, flops=None, like_bytes=None, like_flops=None, like=""):
        e = {"us": round(t_new, 1), "like": like, "like_us": round(t_like, 1)}
        if nbytes:
            e["hbm_frac"] = round(nbytes / t_new / 1e3 / pk["hbm_gbs"], 3)
            e["like_hbm_frac"] = round((like_bytes or nbytes) / t_like / 1e3 / pk["hbm_gbs"], 3)
        if flops:
            e["tensor_frac"] = round(flops / t_new / 1e6 / pk["bf16_tflops"], 4)
            e["like_tensor_frac"] = round((like_flops or flops) / t_like / 1e6 / pk["bf16_tflops"], 4)
        out[name] = e

    # norms: 32,768 rows (the stream alone is past the L2)
    rows = 32768
    res, dl = rnd(rows, d), rnd(rows, d)
    w = [rnd(d) for _ in range(4)]
    o1, o2 = torch.empty(rows, d, dtype=bf, device=dev), torch.empty(rows, d, dtype=bf, device=dev)
    t_new = us(lambda: ops.add_layernorm(res, dl, None, w[0], w[1], o1, 1e-6, None, w[2], w[3], o2))
    t_like = us(lambda: (ops.add_rmsnorm(res, dl, w[0], o1, 1e-6), ops.add_rmsnorm(res, None, w[2], o2, 1e-6)))
    entry("add_layernorm_two_outputs", t_new, t_like, rows * d * (4 + 4 + 4 + 2 + 2), like_bytes=rows * d * (4 + 4 + 4 + 2 + 4 + 2),
          like="add_rmsnorm twice (the two norms of a layer)")
    del res, dl, o1, o2
    # gating: 16,384 rows of the feed-forward's width
    rows = 16384
    gu32, gu16 = rnd(rows, 2 * inter), rnd(rows, 2 * inter, dt=bf)
    h = torch.empty(rows, inter, dtype=bf, device=dev)
    t_new = us(lambda: ops.glu_clamped(gu32, h, 7.0, 1.702, 1.0))
    t_like = us(lambda: ops.silu_mul(gu16, h))
    entry("glu_clamped", t_new, t_like, rows * inter * (8 + 2), like_bytes=rows * inter * (4 + 2), like="silu_mul (bfloat16 in)")
    del gu32, gu16, h
    # attention: decoding rows (64 rows at 4,096 keys: the cache alone is past the L2) and one prompt of 4,096 tokens
    page, ctx, b = PAGE, 4096, 64
    pages = b * ctx // page
    table = torch.arange(pages, dtype=torch.int32, device=dev).view(b, -1).contiguous()
    sinks = rnd(hq)
    for name, dk, dv, vw, h_kv, window in (("sink_attention", hd, hd, hd, hkv, None), ("latent_attention", 4 * hd + hd // 2, 4 * hd, 0, 1, 1024)):
        kp = rnd(pages, h_kv, page, dk, dt=bf)
        vp = kp if not vw else rnd(pages, h_kv, page, dv, dt=bf)
        q = rnd(b, hq * dk)
        o = torch.empty(b, hq * dv, dtype=bf, device=dev)
        pos = torch.full((b,), ctx - 1, dtype=torch.int32, device=dev)
        slot = torch.arange(b, dtype=torch.int32, device=dev)
        sk = sinks if vw else None
        seen = min(ctx, window or ctx)
        items = b * h_kv * (-(-(hq // h_kv) // 16))
        splits = max(1, min(6 * 148 // items, -(-seen // 64), 32))  # (the engine's rule: parts/wide_attend.py)
        scratch = torch.empty(max(1, ops.attention_wide_mma_scratch_words(items, dv, splits)), device=dev)
        t_new = us(lambda: ops.attention_wide_mma(q, kp, vp, o, sk, pos, slot, table, None, None, b, True, hq, h_kv, dk, dv, window, 0.1,
                                                  splits, scratch))
        t_exact = us(lambda: ops.attention_wide(q, kp, vp, o, sk, pos, slot, table, hq, h_kv, dk, dv, window, 0.1), reps=2)
        nbytes = b * seen * h_kv * (dk + (dv if vw else 0)) * 2
        if vw:  # keys and values of one width: the engine sends decoding rows to the cluster kernel, with the sink in its merges
            from types import SimpleNamespace

            from machserve_b200.parts.attention import decode_launch

            q16, o16 = q.to(bf), torch.empty(b, hq * hd, dtype=bf, device=dev)
            sp, stg, wr, kpw, parts = decode_launch(SimpleNamespace(sm_count=ops.sm_count()), hd, ops.attention_decode_cluster_max_stages(hd),
                                                    {}, b * hkv, -(-ctx // 64))
            cl = lambda sinks_: ops.attention_decode_cluster(q16, kp, vp, o16, pos, slot, table, hq, hkv, hd, None, 0.1, sp, stg, warps=wr,
                                                             keys_per_warp=kpw, parts=1, sinks=sinks_)
            t_sink, t_like = us(lambda: cl(sk)), us(lambda: cl(None))
            entry(name + "_decode", t_sink, t_like, nbytes, like="attention_decode_cluster without a sink")
            out[name + "_decode"]["mma_kernel_us"] = round(t_new, 1)  # (what other widths get)
        else:
            entry(name + "_decode", t_new, t_new, nbytes, like="(no like kernel: one plane read for keys and values)")
        out[name + "_decode"]["exact_kernel_us"] = round(t_exact, 1)
        # one prompt of 4,096 tokens in one step, in tiles of 64, 32 or 16 rows
        n = ctx
        posp = torch.arange(n, dtype=torch.int32, device=dev)
        slotp = torch.zeros(n, dtype=torch.int32, device=dev)
        qp, op = rnd(n, hq * dk), torch.empty(n, hq * dv, dtype=bf, device=dev)
        tile = ops.attention_wide_mma_tile_rows(dv)
        u0 = torch.arange(0, n, tile, dtype=torch.int32, device=dev)
        un = torch.full_like(u0, tile)
        t_new = us(lambda: ops.attention_wide_mma(qp, kp, vp, op, sk, posp, slotp, table, u0, un, u0.numel(), False, hq, h_kv, dk, dv, window, 0.1),
                   reps=2)
        t_exact = us(lambda: ops.attention_wide(qp, kp, vp, op, sk, posp, slotp, table, hq, h_kv, dk, dv, window, 0.1, share_rows=True), reps=1)
        pairs = n * (n + 1) // 2 if not window else sum(min(p + 1, window) for p in range(n))
        flops = 2 * pairs * hq * (dk + dv)
        if vw and ops.attention_prefill_tc_supports(hd, page):
            # at key and value rows of 64 or 128 the engine sends portions to the tcgen05 kernel, with the sink in its finish
            qp16, op16 = qp.to(bf), torch.empty(n, hq * hd, dtype=bf, device=dev)
            t0 = torch.arange(0, n, 128, dtype=torch.int32, device=dev)
            tn = torch.full_like(t0, 128)
            tiles = t0.numel()
            splits_p, alone, run_tiles = ops.attention_prefill_tc_plan(tiles, hq, hkv, hd, n, tiles * (tiles + 1) // 2)
            words = ops.attention_prefill_tc_scratch_words(tiles, hq, hd, splits_p)
            scr = torch.zeros(max(words, 1), dtype=torch.float32, device=dev) if words else None
            counters = torch.zeros(tiles * hq, dtype=torch.int32, device=dev) if words else None
            tc = lambda sinks_: ops.attention_prefill_tc(qp16, kp, vp, op16, t0, tn, tiles, posp, slotp, table, hq, hkv, hd, None, 0.1,
                                                         splits_p, scr, counters, alone=alone, run_tiles=run_tiles, sinks=sinks_)
            t_sink, t_like = us(lambda: tc(sk), reps=2), us(lambda: tc(None), reps=2)
            entry(name + "_prefill", t_sink, t_like, flops=flops, like="attention_prefill_tc (tcgen05) without a sink")
            out[name + "_prefill"]["mma_kernel_us"] = round(t_new, 1)  # (what other widths get)
        else:
            entry(name + "_prefill", t_new, t_new, flops=flops, like="(no like kernel)")
        out[name + "_prefill"]["exact_kernel_us"] = round(t_exact, 1)
        del kp, vp, q, o, qp, op
    # between the input product and the attention: 16,384 rows
    rows = 16384
    pos = (torch.arange(rows, dtype=torch.int32, device=dev) % 4096).contiguous()
    slot = (torch.arange(rows, dtype=torch.int32, device=dev) // 4096).contiguous()
    pages = rows // page
    table = torch.arange(pages, dtype=torch.int32, device=dev).view(4, -1).contiguous()
    qkvw = (hq + 2 * hkv) * hd
    proj = rnd(rows, qkvw)
    kp, vp = torch.zeros(pages, hkv, page, hd, dtype=bf, device=dev), torch.zeros(pages, hkv, page, hd, dtype=bf, device=dev)
    qo = torch.empty(rows, hq * hd, device=dev)
    t_new = us(lambda: ops.qk_norm_store(proj, w[0].new_ones(hq * hd), w[0].new_ones(hkv * hd), 1e-6, 0.1, 1024, pos, slot, table, qo, kp, vp, hkv, hd, hd))
    proj16, qo16 = proj.to(bf), torch.empty(rows, hq * hd, dtype=bf, device=dev)
    ang = torch.zeros(4096, hd // 2, 2, device=dev)
    t_like = us(lambda: ops.rope_kv_store(proj16, None, pos, slot, table, ang, hd, False, qo16, kp, vp, hq, hkv, hd))
    entry("qk_norm_store", t_new, t_like, rows * (qkvw * 4 + hq * hd * 4 + 2 * hkv * hd * 2), like_bytes=rows * (qkvw * 2 + hq * hd * 2 + 2 * hkv * hd * 2),
          like="rope_kv_store (bfloat16 in and out)")
    return out


def workload_venarax(a, pk):
    """The Venarax design at the layer sizes of the Qwen2.5 shapes, beside the dense decoder at the same sizes: decode
    at the headline batch and context, one prompt of `--prefill` tokens, and the new kernels alone."""
    import torch

    from machserve_b200 import ops

    out = {}
    shapes = sorted(SHAPES) if a.venarax_shapes == "all" else [x.strip() for x in a.venarax_shapes.split(",") if x.strip()]
    for shape in shapes:
        raw = SHAPES[shape]
        layers = min(raw["num_hidden_layers"], a.layers or 12)  # (layers of equal sizes: twelve tell what all tell)
        res = {"layers": layers}
        steps = max(10, a.steps // 2)
        for which in ("venarax", "dense"):
            kw = dict(config=venarax_config(raw, layers), vocab=raw["vocab_size"]) if which == "venarax" else {}
            b = DecodeBench(a, raw, layers, "bf16", a.batch, a.context + 4 * (steps + a.warmup) + a.batch + 64, **kw)
            times, launches = b.time_decode(a.batch, a.context, steps, a.warmup, blocks=3, sampled=False)
            pms = b.time_prefill(a.prefill, 2, reps=3)
            res[which] = {"decode_ms_per_step": round(times[len(times) // 2], 4), "decode_tokens_per_s": round(a.batch * 1000.0 / times[len(times) // 2], 1),
                          "launches_per_step": launches // steps, "prefill_ms": round(pms, 3), "prefill_tokens_per_s": round(a.prefill * 1000.0 / pms, 1)}
            b.runner.check_device_status()
            b.release_all()
            del b
            free_device_memory()
        if not a.no_points:
            res["kernels"] = time_venarax_kernels(torch, ops, raw, pk)
        free_device_memory()
        out[shape] = res
    return {"batch": a.batch, "context": a.context, "prefill_tokens": a.prefill, "dtype": "bf16",
            "data": "random-init weights drawn on the device, seeded uniform random token ids", "peaks": pk["source"], "sizes": out}


def fozutar_config(raw, layers, chunk=1024):
    """A Fozutar configuration with the layer sizes of the Qwen2 shape `raw`: the same width, heads, key heads, head size
    and vocabulary; every third layer an attention layer (chunks of `chunk` positions, a bias table of 32 rows that
    reaches 4,096), the others gated linear attention with half as many heads of twice the value size (keys half the width,
    values the whole width, a decay projection of rank 16); the feed-forwards dense (the shape's own size) and routed (eight
    experts of half that size, two a token: the same multiply-adds a token) in turn; no loop."""
    d, i, v, hq, hkv, hd = sizes(raw)
    att = {"type": "attention", "mixer": {"heads": hq, "kv_heads": hkv, "dim": hd, "vdim": hd, "scale": hd ** -0.5, "softcap": 50.0,
                                          "bias_rows": 32, "bias_max": 4096, "mask": {"size": chunk}}}
    gla = {"type": "gla", "mixer": {"heads": max(1, hq // 2), "dim": hd, "vdim": 2 * hd, "tau": 16.0, "decay_rank": 16}}
    dense = {"kind": "dense", "ff": i}
    moe = {"kind": "moe", "expert": {"ff": i // 2 // 32 * 32}, "router": {"experts": 8, "top": 2}}
    return {"architecture": "Fozutar", "vocab": v, "width": d, "max_positions": 8192, "norm": {"eps": 1e-6}, "embedding": {"scale": 1.0},
            "layers": [{**(att if n % 3 == 2 else gla), "mlp": moe if n % 2 else dense} for n in range(layers)]}


def time_fozutar_kernels(torch, ops, raw, pk):
    """The Fozutar design's kernels alone, each beside the like kernel of the dense decoder at equal sizes where there is
    one (inputs larger than the L2; a CUDA graph of a few launches between events)."""
    d, inter, _, hq, hkv, hd = sizes(raw)
    dev, bf = "cuda:0", torch.bfloat16
    g = torch.Generator(device=dev).manual_seed(0)
    rnd = lambda *shape, dt=torch.float32, scale=1.0: (torch.randn(*shape, device=dev, generator=g) * scale).to(dt)

    def us(fn, reps=5):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            for _ in range(reps):
                fn()
        graph.replay()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        graph.replay()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / reps * 1000

    out = {}

    def entry(name, t_new, t_like=None, nbytes=None, flops=None, like_bytes=None, like_flops=None, like="(no like kernel)"):
        e = {"us": round(t_new, 1), "like": like}
        if t_like is not None:
            e["like_us"] = round(t_like, 1)
        if nbytes:
            e["hbm_frac"] = round(nbytes / t_new / 1e3 / pk["hbm_gbs"], 3)
            if t_like is not None:
                e["like_hbm_frac"] = round((like_bytes or nbytes) / t_like / 1e3 / pk["hbm_gbs"], 3)
        if flops:
            e["tensor_frac"] = round(flops / t_new / 1e6 / pk["bf16_tflops"], 4)
            if t_like is not None:
                e["like_tensor_frac"] = round((like_flops or flops) / t_like / 1e6 / pk["bf16_tflops"], 4)
        out[name] = e

    # the norm that adds a layer's two halves: 32,768 rows
    rows = 32768
    res, da, db = rnd(rows, d), rnd(rows, d), rnd(rows, d)
    w = rnd(d)
    o1 = torch.empty(rows, d, dtype=bf, device=dev)
    t_new = us(lambda: ops.add_streams_rmsnorm(res, da, db, None, None, w, o1, 1e-6))
    t_like = us(lambda: ops.add_rmsnorm(res, da, w, o1, 1e-6))
    entry("add_streams_rmsnorm", t_new, t_like, rows * d * (4 + 4 + 4 + 4 + 2), like_bytes=rows * d * (4 + 4 + 4 + 2), like="add_rmsnorm (one delta)")
    del res, da, db, o1
    # gating: 16,384 rows of the feed-forward's width
    rows = 16384
    gu16 = rnd(rows, 2 * inter, dt=bf)
    h = torch.empty(rows, inter, dtype=bf, device=dev)
    t_new = us(lambda: ops.gated_act_mul(gu16, h, "gelu_tanh"))
    t_like = us(lambda: ops.silu_mul(gu16, h))
    entry("gated_act_mul_gelu", t_new, t_like, rows * inter * 6, like="silu_mul")
    del gu16, h
    # between the input product and the attention: 16,384 rows
    page = PAGE
    pos = (torch.arange(rows, dtype=torch.int32, device=dev) % 4096).contiguous()
    slot = (torch.arange(rows, dtype=torch.int32, device=dev) // 4096).contiguous()
    pages = rows // page
    table = torch.arange(pages, dtype=torch.int32, device=dev).view(4, -1).contiguous()
    proj = rnd(rows, (hq + hkv) * hd)
    kp, vp = torch.zeros(pages, hkv, page, hd, dtype=bf, device=dev), torch.zeros(pages, hkv, page, hd, dtype=bf, device=dev)
    qo = torch.empty(rows, hq * hd, device=dev)
    t_new = us(lambda: ops.head_norm_store(proj, 1e-6, pos, slot, table, qo, kp, vp, hq, hkv, hd, hd, None))
    proj16, qo16 = rnd(rows, (hq + 2 * hkv) * hd, dt=bf), torch.empty(rows, hq * hd, dtype=bf, device=dev)
    ang = torch.zeros(4096, hd // 2, 2, device=dev)
    t_like = us(lambda: ops.rope_kv_store(proj16, None, pos, slot, table, ang, hd, False, qo16, kp, vp, hq, hkv, hd))
    entry("head_norm_store", t_new, t_like, rows * ((hq + hkv) * hd * 4 + hq * hd * 4 + 2 * hkv * hd * 2),
          like_bytes=rows * ((hq + 2 * hkv) * hd * 2 + hq * hd * 2 + 2 * hkv * hd * 2), like="rope_kv_store (bfloat16 in and out)")
    del proj, proj16, qo, qo16, kp, vp
    # attention with cap, bias and chunks of 1,024: 64 decoding rows at 4,096 tokens, and one prompt of 4,096 tokens
    from machserve_b200.parts.chunked_attention import bias_by_distance

    chunk, ctx, b = 1024, 4096, 64
    pages = b * ctx // page
    table = torch.arange(pages, dtype=torch.int32, device=dev).view(b, -1).contiguous()
    kp, vp = rnd(pages, hkv, page, hd, dt=bf), rnd(pages, hkv, page, hd, dt=bf)
    score = ops.ScoreExtras(50.0, bias_by_distance(torch.randn(32, hq), 4096, chunk).to(dev), chunk)
    q = rnd(b, hq * hd)
    o = torch.empty(b, hq * hd, dtype=bf, device=dev)
    posd = torch.full((b,), ctx - 1, dtype=torch.int32, device=dev)
    slotd = torch.arange(b, dtype=torch.int32, device=dev)
    items = b * hkv * (-(-(hq // hkv) // 16))
    splits = max(1, min(6 * 148 // items, -(-(chunk + 63) // 64), 32))
    scratch = torch.empty(max(1, ops.attention_wide_mma_scratch_words(items, hd, splits)), device=dev)
    t_new = us(lambda: ops.attention_wide_mma(q, kp, vp, o, None, posd, slotd, table, None, None, b, True, hq, hkv, hd, hd, None, 0.1, splits,
                                              scratch, score=score))
    from types import SimpleNamespace

    from machserve_b200.parts.attention import decode_launch

    q16 = q.to(bf)
    sp, stg, wr, kpw, parts = decode_launch(SimpleNamespace(sm_count=ops.sm_count()), hd, ops.attention_decode_cluster_max_stages(hd), {},
                                            b * hkv, -(-chunk // 64))
    t_like = us(lambda: ops.attention_decode_cluster(q16, kp, vp, o, posd, slotd, table, hq, hkv, hd, chunk, 0.1, sp, stg, warps=wr,
                                                     keys_per_warp=kpw, parts=1))
    entry("chunked_attention_decode", t_new, t_like, b * chunk * hkv * 2 * hd * 2, like="attention_decode_cluster under a window of 1,024")
    n = ctx
    posp = torch.arange(n, dtype=torch.int32, device=dev)
    slotp = torch.zeros(n, dtype=torch.int32, device=dev)
    qp, op = rnd(n, hq * hd), torch.empty(n, hq * hd, dtype=bf, device=dev)
    tile = ops.attention_wide_mma_tile_rows(hd)
    u0 = torch.arange(0, n, tile, dtype=torch.int32, device=dev)
    un = torch.full_like(u0, tile)
    t_new = us(lambda: ops.attention_wide_mma(qp, kp, vp, op, None, posp, slotp, table, u0, un, u0.numel(), False, hq, hkv, hd, hd, None, 0.1,
                                              score=score), reps=2)
    pairs = sum(p % chunk + 1 for p in range(n))
    flops = 4 * pairs * hq * hd
    t_like, like_flops = None, None
    if ops.attention_prefill_tc_supports(hd, page):
        qp16 = qp.to(bf)
        t0 = torch.arange(0, n, 128, dtype=torch.int32, device=dev)
        tn = torch.full_like(t0, 128)
        tiles = t0.numel()
        splits_p, alone, run_tiles = ops.attention_prefill_tc_plan(tiles, hq, hkv, hd, chunk + 128, tiles * 9)
        words = ops.attention_prefill_tc_scratch_words(tiles, hq, hd, splits_p)
        scr = torch.zeros(max(words, 1), dtype=torch.float32, device=dev) if words else None
        counters = torch.zeros(tiles * hq, dtype=torch.int32, device=dev) if words else None
        t_like = us(lambda: ops.attention_prefill_tc(qp16, kp, vp, op, t0, tn, tiles, posp, slotp, table, hq, hkv, hd, chunk, 0.1, splits_p,
                                                     scr, counters, alone=alone, run_tiles=run_tiles), reps=2)
        like_flops = 4 * sum(min(p + 1, chunk) for p in range(n)) * hq * hd
    entry("chunked_attention_prefill", t_new, t_like, flops=flops, like_flops=like_flops,
          like="attention_prefill_tc (tcgen05) under a window of 1,024" if t_like else "(no like kernel)")
    del kp, vp, q, o, qp, op
    # the recurrence: 64 sequences of one token (the states alone are past the L2 at the larger shapes), and one of 4,096
    heads, dk, dv = max(1, hq // 2), hd, 2 * hd
    kw, vw = heads * dk, heads * dv
    state = torch.zeros(b, heads, dk, dv, device=dev)
    proj = rnd(n, 2 * kw + 2 * vw + 16, scale=0.1)
    dec = torch.exp(-torch.rand(n, kw, device=dev, generator=g) * 0.1)
    og = torch.empty(n, vw, device=dev)
    cu1 = torch.arange(b + 1, dtype=torch.int32, device=dev)
    t_new = us(lambda: ops.gla_scan(proj[:b], 0, kw, 2 * kw, dec[:b], 0.1, state, cu1, slotd, slotd, og[:b], b, heads, dk, dv))
    entry("gla_scan_decode", t_new, nbytes=2 * b * heads * dk * dv * 4)
    cup = torch.tensor([0, n], dtype=torch.int32, device=dev)
    zero = torch.zeros(n, dtype=torch.int32, device=dev)
    t_new = us(lambda: ops.gla_scan(proj, 0, kw, 2 * kw, dec, 0.1, state, cup, zero[:1], zero, og, 1, heads, dk, dv, narrow=True), reps=2)
    entry("gla_scan_prefill", t_new, flops=n * heads * dk * dv * 4)  # (CUDA-core multiply-adds: the scan is sequential)
    w2 = rnd(kw, 16, dt=bf)
    y = torch.empty(n, vw, dtype=bf, device=dev)
    normw = rnd(dv)
    t_new = us(lambda: (ops.gla_decay(proj[:, 2 * kw + 2 * vw:], w2, None, 16.0, dec), ops.gla_output(og, proj[:, 2 * kw + vw: 2 * kw + 2 * vw], normw, 1e-6, y, heads, dv)))
    entry("gla_decay_and_output", t_new, nbytes=n * (16 * 4 + kw * 4 + vw * 4 + vw * 4 + vw * 2))
    del state, proj, dec, og, y
    # the routed feed-forward: eight experts of half the dense size, two a token; 8 decoding rows and 4,096 rows of a prompt
    experts, top, ff = 8, 2, inter // 2 // 32 * 32
    wg, wu, wd = rnd(experts, ff, d, dt=bf, scale=0.02), rnd(experts, ff, d, dt=bf, scale=0.02), rnd(experts, d, ff, dt=bf, scale=0.02)
    for t, name in ((8, "routed_experts_decode"), (4096, "routed_experts_prefill")):
        x = rnd(t, d, dt=bf)
        logits = rnd(t, experts)
        ids, weights = torch.empty(t, top, dtype=torch.int32, device=dev), torch.empty(t, top, device=dev)
        ops.moe_route(logits, top, ids, weights)
        hbuf = torch.empty(t * top, ff, dtype=bf, device=dev)
        yb = torch.empty(t, d, device=dev)
        slots = torch.zeros(t, dtype=torch.int32, device=dev)
        w_dense = rnd(2 * inter, d, dt=bf, scale=0.02)
        w_down = rnd(d, inter, dt=bf, scale=0.02)
        gu = torch.empty(t, 2 * inter, dtype=bf, device=dev)
        hd_ = torch.empty(t, inter, dtype=bf, device=dev)
        od = torch.empty(t, d, dtype=bf, device=dev)
        if t <= 16:
            t_new = us(lambda: (ops.moe_route(logits, top, ids, weights), ops.moe_gate_up_pairs(x, wg, wu, ids, slots, hbuf, "silu"),
                                ops.moe_down_pairs(hbuf, wd, ids, weights, slots, yb)))
            t_like = us(lambda: (ops.gemm_small_m_silu_mul(x, w_dense[:inter], w_dense[inter:], hd_), ops.linear(hd_, w_down, None, od)))
            touched = min(experts, t * top)
            scratch = torch.empty(ops.moe_grouped_scratch_ints(t * top, experts), dtype=torch.int32, device=dev)
            z = torch.empty(t * top, d, device=dev)
            t_tiles = us(lambda: (ops.moe_route(logits, top, ids, weights), ops.moe_grouped(x, wg, wu, wd, ids, weights, slots, scratch, hbuf, z, yb, "silu")))
            entry(name, t_new, t_like, nbytes=touched * 3 * ff * d * 2, like_bytes=3 * inter * d * 2,
                  like="the dense gated feed-forward of the same multiply-adds a token (few-row products)")
            out[name]["sorted_tiles_us"] = round(t_tiles, 1)  # (the form for many rows, at these few)
        else:
            scratch = torch.empty(ops.moe_grouped_scratch_ints(t * top, experts), dtype=torch.int32, device=dev)
            z = torch.empty(t * top, d, device=dev)
            t_new = us(lambda: (ops.moe_route(logits, top, ids, weights), ops.moe_grouped(x, wg, wu, wd, ids, weights, slots, scratch, hbuf, z, yb, "silu")), reps=2)
            t_like = us(lambda: (ops.linear(x, w_dense, None, gu), ops.silu_mul(gu, hd_), ops.linear(hd_, w_down, None, od)), reps=2)
            entry(name, t_new, t_like, flops=6 * t * top * ff * d, like_flops=6 * t * inter * d,
                  like="the dense gated feed-forward of the same multiply-adds a token (library products)")
    return out


def workload_fozutar(a, pk):
    """The Fozutar design at the layer sizes of the Qwen2.5 shapes, beside the dense decoder at the same sizes: decode
    at the headline batch and context, one prompt of `--prefill` tokens, and the new kernels alone."""
    import torch

    from machserve_b200 import ops

    out = {}
    shapes = sorted(SHAPES) if a.fozutar_shapes == "all" else [x.strip() for x in a.fozutar_shapes.split(",") if x.strip()]
    for shape in shapes:
        raw = SHAPES[shape]
        layers = min(raw["num_hidden_layers"], a.layers or 12)  # (layers of like sizes: twelve tell what all tell)
        res = {"layers": layers}
        steps = max(10, a.steps // 2)
        for which in ("fozutar", "dense"):
            kw = dict(config=fozutar_config(raw, layers), vocab=raw["vocab_size"]) if which == "fozutar" else {}
            b = DecodeBench(a, raw, layers, "bf16", a.batch, a.context + 4 * (steps + a.warmup) + a.batch + 64, **kw)
            times, launches = b.time_decode(a.batch, a.context, steps, a.warmup, blocks=3, sampled=False)
            pms = b.time_prefill(a.prefill, 2, reps=3)
            res[which] = {"decode_ms_per_step": round(times[len(times) // 2], 4), "decode_tokens_per_s": round(a.batch * 1000.0 / times[len(times) // 2], 1),
                          "launches_per_step": launches // steps, "prefill_ms": round(pms, 3), "prefill_tokens_per_s": round(a.prefill * 1000.0 / pms, 1)}
            b.runner.check_device_status()
            b.release_all()
            del b
            free_device_memory()
        if not a.no_points:
            res["kernels"] = time_fozutar_kernels(torch, ops, raw, pk)
        free_device_memory()
        out[shape] = res
    return {"batch": a.batch, "context": a.context, "prefill_tokens": a.prefill, "dtype": "bf16",
            "data": "random-init weights drawn on the device, seeded uniform random token ids", "peaks": pk["source"], "sizes": out}


def modadra_config(raw, layers, window=1024):
    """A Modadra configuration with the layer sizes of the Qwen2 shape `raw`: the same width, vocabulary, heads, key heads
    and head size on the attention side (keys and values of the head size, half of every head rotated, a window of `window`
    positions); beside it a gated delta rule with half as many value heads of twice the head size, a key head for every
    two of them and a convolution of four taps; every layer's feed-forward routed (eight experts in four groups of which two
    are kept, two experts a token, each half the shape's size: the same multiply-adds a token as a gated dense one of that
    size has in two of its three matrices)."""
    d, i, v, hq, hkv, hd = sizes(raw)
    heads = max(1, hq // 2)
    kv = heads // 2 if heads % 2 == 0 else heads
    left = {"heads": hq, "kv_heads": hkv, "dim": hd, "vdim": hd, "scale": hd ** -0.5, "rot": {"dims": hd // 2, "base": 10000.0},
            "mask": {"size": window}}
    right = {"heads": heads, "kv_heads": kv, "dim": hd, "vdim": 2 * hd, "conv": 4}
    moe = {"kind": "moe", "expert": {"ff": i // 2 // 32 * 32}, "router": {"experts": 8, "top": 2, "scale": 1.5, "groups": {"count": 4, "keep": 2}}}
    return {"architecture": "Modadra", "vocab": v, "width": d, "max_positions": 8192, "norm": {"eps": 1e-6}, "residual_mult": 0.5,
            "logit_softcap": 30.0, "layers": [{"type": "parallel", "mixer": {"left": left, "right": right}, "mlp": moe} for _ in range(layers)]}


def time_modadra_kernels(torch, ops, raw, pk):
    """The Modadra design's kernels alone, each beside the like kernel of the closest designs at equal sizes where there is
    one (inputs larger than the L2; a CUDA graph of a few launches between events)."""
    d, inter, _, hq, hkv, hd = sizes(raw)
    dev, bf = "cuda:0", torch.bfloat16
    g = torch.Generator(device=dev).manual_seed(0)
    rnd = lambda *shape, dt=torch.float32, scale=1.0: (torch.randn(*shape, device=dev, generator=g) * scale).to(dt)

    def us(fn, reps=5):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            for _ in range(reps):
                fn()
        graph.replay()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        graph.replay()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / reps * 1000

    out = {}

    def entry(name, t_new, t_like=None, nbytes=None, flops=None, like_bytes=None, like_flops=None, like="(no like kernel)"):
        e = {"us": round(t_new, 1), "like": like}
        if t_like is not None:
            e["like_us"] = round(t_like, 1)
        if nbytes:
            e["hbm_frac"] = round(nbytes / t_new / 1e3 / pk["hbm_gbs"], 3)
            if t_like is not None:
                e["like_hbm_frac"] = round((like_bytes or nbytes) / t_like / 1e3 / pk["hbm_gbs"], 3)
        if flops:
            e["tensor_frac"] = round(flops / t_new / 1e6 / pk["bf16_tflops"], 4)
            if t_like is not None:
                e["like_tensor_frac"] = round((like_flops or flops) / t_like / 1e6 / pk["bf16_tflops"], 4)
        out[name] = e

    # the mean of the two mixers' normed outputs: 32,768 rows
    rows = 32768
    da, db, res = rnd(rows, d), rnd(rows, d), rnd(rows, d)
    w = rnd(d)
    o32, o16 = torch.empty(rows, d, device=dev), torch.empty(rows, d, dtype=bf, device=dev)
    t_new = us(lambda: ops.norm_pair_mean(da, db, w, w, o32, 1e-6, 0.5))
    t_like = us(lambda: ops.add_rmsnorm(res, da, w, o16, 1e-6))
    entry("norm_pair_mean", t_new, t_like, rows * d * 12, like_bytes=rows * d * (4 + 4 + 4 + 2), like="add_rmsnorm (one delta)")
    del da, db, res, o32, o16
    # between the input product and the attention: 16,384 rows; the head gates after it
    rows, page = 16384, PAGE
    pos = (torch.arange(rows, dtype=torch.int32, device=dev) % 4096).contiguous()
    slot = (torch.arange(rows, dtype=torch.int32, device=dev) // 4096).contiguous()
    pages = rows // page
    table = torch.arange(pages, dtype=torch.int32, device=dev).view(4, -1).contiguous()
    proj = rnd(rows, (hq + 2 * hkv) * hd + hq)
    kp, vp = torch.zeros(pages, hkv, page, hd, dtype=bf, device=dev), torch.zeros(pages, hkv, page, hd, dtype=bf, device=dev)
    qo, qh = torch.empty(rows, hq * hd, device=dev), torch.empty(rows, hq * hd, dtype=bf, device=dev)
    half = torch.zeros(4096, hd // 4, 2, device=dev)
    t_new = us(lambda: ops.rope_store(proj, half, hd // 2, False, pos, slot, table, qo, kp, vp, hq, hkv, hd, hd, q_half=qh))
    proj16, qo16 = rnd(rows, (hq + 2 * hkv) * hd, dt=bf), torch.empty(rows, hq * hd, dtype=bf, device=dev)
    ang = torch.zeros(4096, hd // 2, 2, device=dev)
    t_like = us(lambda: ops.rope_kv_store(proj16, None, pos, slot, table, ang, hd, False, qo16, kp, vp, hq, hkv, hd))
    entry("rope_store", t_new, t_like, rows * ((hq + 2 * hkv) * hd * 4 + hq * hd * 6 + 2 * hkv * hd * 2),
          like_bytes=rows * ((hq + 2 * hkv) * hd * 2 + hq * hd * 2 + 2 * hkv * hd * 2), like="rope_kv_store (bfloat16 in and out)")
    gate = proj[:, (hq + 2 * hkv) * hd:]
    t_new = us(lambda: ops.head_gate_mul(qh, gate, qh, hq, hd))
    gu16 = rnd(rows, 2 * hq * hd, dt=bf)
    t_like = us(lambda: ops.silu_mul(gu16, qo16))
    entry("head_gate_mul", t_new, t_like, rows * hq * hd * 4, like_bytes=rows * hq * hd * 6, like="silu_mul")
    del proj, proj16, qo, qo16, qh, kp, vp, gu16
    # attention with the one more in the denominator under a window of 1,024: 64 decoding rows at 4,096 tokens and one prompt
    # of 4,096 tokens, each on the kernel that the dense decoder uses, with and without the sink
    from types import SimpleNamespace

    from machserve_b200.parts.attention import decode_launch

    window, ctx, b = 1024, 4096, 64
    pages = b * ctx // page
    table = torch.arange(pages, dtype=torch.int32, device=dev).view(b, -1).contiguous()
    kp, vp = rnd(pages, hkv, page, hd, dt=bf), rnd(pages, hkv, page, hd, dt=bf)
    sinks = torch.zeros(hq, device=dev)
    q16 = rnd(b, hq * hd, dt=bf)
    o = torch.empty(b, hq * hd, dtype=bf, device=dev)
    posd = torch.full((b,), ctx - 1, dtype=torch.int32, device=dev)
    slotd = torch.arange(b, dtype=torch.int32, device=dev)
    if ops.attention_decode_supports(hd, hq // hkv):
        sp, stg, wr, kpw, parts = decode_launch(SimpleNamespace(sm_count=ops.sm_count()), hd, ops.attention_decode_cluster_max_stages(hd), {},
                                                b * hkv, -(-window // 64) + 1)
        run = lambda sk: ops.attention_decode_cluster(q16, kp, vp, o, posd, slotd, table, hq, hkv, hd, window, 0.1, sp, stg, warps=wr,
                                                      keys_per_warp=kpw, parts=1, sinks=sk)
        t_new, t_like = us(lambda: run(sinks)), us(lambda: run(None))
        entry("sink_window_attention_decode", t_new, t_like, b * window * hkv * 2 * hd * 2, like="the same kernel without the sink")
    n = ctx
    posp = torch.arange(n, dtype=torch.int32, device=dev)
    slotp = torch.zeros(n, dtype=torch.int32, device=dev)
    if ops.attention_prefill_tc_supports(hd, page):
        qp16, op = rnd(n, hq * hd, dt=bf), torch.empty(n, hq * hd, dtype=bf, device=dev)
        t0 = torch.arange(0, n, 128, dtype=torch.int32, device=dev)
        tn = torch.full_like(t0, 128)
        tiles = t0.numel()
        splits_p, alone, run_tiles = ops.attention_prefill_tc_plan(tiles, hq, hkv, hd, window + 128, tiles * 9)
        words = ops.attention_prefill_tc_scratch_words(tiles, hq, hd, splits_p)
        scr = torch.zeros(max(words, 1), dtype=torch.float32, device=dev) if words else None
        counters = torch.zeros(tiles * hq, dtype=torch.int32, device=dev) if words else None
        run = lambda sk: ops.attention_prefill_tc(qp16, kp, vp, op, t0, tn, tiles, posp, slotp, table, hq, hkv, hd, window, 0.1, splits_p,
                                                  scr, counters, alone=alone, run_tiles=run_tiles, sinks=sk)
        t_new, t_like = us(lambda: run(sinks), reps=2), us(lambda: run(None), reps=2)
        flops = 4 * sum(min(p + 1, window) for p in range(n)) * hq * hd
        entry("sink_window_attention_prefill", t_new, t_like, flops=flops, like="the same tcgen05 kernel without the sink")
        del qp16, op
    del kp, vp, q16, o
    # the recurrence: what it reads from the input product (4,096 rows), 64 sequences of one token, and one sequence of 4,096
    heads = max(1, hq // 2)
    kv = heads // 2 if heads % 2 == 0 else heads
    dk, dv, taps = hd, 2 * hd, 4
    kw, vw = kv * dk, heads * dv
    ch = 2 * kw + vw
    width = ch + vw + 2 * heads
    conv_off = heads * dk * dv
    state = torch.zeros(b, conv_off + (taps - 1) * ch, device=dev)
    proj = rnd(n, width, scale=0.3)
    conv_w, a_log, dt_bias = rnd(ch, taps, scale=0.5), rnd(heads, scale=0.3), rnd(heads, scale=0.3)
    qkv, bg = torch.empty(n, ch, device=dev), torch.empty(n, 2 * heads, device=dev)
    cup = torch.tensor([0, n], dtype=torch.int32, device=dev)
    zero = torch.zeros(n, dtype=torch.int32, device=dev)
    t_new = us(lambda: (ops.gdr_prepare(proj, 0, ch + vw, ch + vw + heads, conv_w, a_log, dt_bias, state, conv_off, cup, zero, zero, qkv, bg,
                                        heads, kv, dk, dv, dk ** -0.5),
                        ops.gdr_conv_update(proj, 0, taps, ch, state, conv_off, cup, zero[:1], zero, 1)))
    gkw, gvw = heads * dk, heads * dv  # (the gated linear attention of the same heads: what it computes between product and scan)
    gproj = rnd(n, 2 * gkw + 2 * gvw + 16, scale=0.1)
    w2 = rnd(gkw, 16, dt=bf)
    dec = torch.empty(n, gkw, device=dev)
    t_like = us(lambda: ops.gla_decay(gproj[:, 2 * gkw + 2 * gvw:], w2, None, 16.0, dec))
    entry("gdr_prepare_and_conv_update", t_new, t_like, n * (ch * 4 * 2 + 2 * heads * 4 * 2), like_bytes=n * (16 * 4 + gkw * 4),
          like="gla_decay (what the gated linear attention computes before its scan)")
    og = torch.empty(n, vw, device=dev)
    cu1 = torch.arange(b + 1, dtype=torch.int32, device=dev)
    t_new = us(lambda: ops.gdr_scan(qkv[:b], bg[:b], state, cu1, slotd, slotd, og[:b], b, heads, kv, dk, dv))
    gstate = torch.zeros(b, heads, dk, dv, device=dev)
    dec.uniform_(0.9, 1.0)
    t_like = us(lambda: ops.gla_scan(gproj[:b], 0, gkw, 2 * gkw, dec[:b], 0.1, gstate, cu1, slotd, slotd, og[:b], b, heads, dk, dv))
    entry("gdr_scan_decode", t_new, t_like, 2 * b * heads * dk * dv * 4, like="gla_scan (decode)")
    t_new = us(lambda: ops.gdr_scan(qkv, bg, state, cup, zero[:1], zero, og, 1, heads, kv, dk, dv, narrow=True), reps=2)
    t_like = us(lambda: ops.gla_scan(gproj, 0, gkw, 2 * gkw, dec, 0.1, gstate, cup, zero[:1], zero, og, 1, heads, dk, dv, narrow=True), reps=2)
    # (CUDA-core multiply-adds, the scan is sequential: three products of the state a token here, two there)
    entry("gdr_scan_prefill", t_new, t_like, flops=n * heads * dk * dv * 6, like_flops=n * heads * dk * dv * 4, like="gla_scan (one prompt)")
    y = torch.empty(n, vw, dtype=bf, device=dev)
    normw = rnd(dv)
    t_new = us(lambda: ops.gla_output(og, proj[:, ch:ch + vw], normw, 1e-6, y, heads, dv))
    entry("gdr_output (gla_output)", t_new, nbytes=n * vw * (4 + 4 + 2), like="the same kernel")
    del state, proj, qkv, bg, og, gproj, dec, gstate, y
    # the soft cap on the logits: 64 rows of the vocabulary
    v = raw["vocab_size"]
    lg = rnd(b, v)
    t_new = us(lambda: ops.softcap(lg, 30.0))
    entry("softcap", t_new, nbytes=b * v * 8)
    del lg
    # the router and the experts without a gate: eight experts, two a token; 8 decoding rows and 4,096 rows of a prompt, beside
    # the gated experts of the same sizes under the softmax router
    experts, top, ff = 8, 2, inter // 2 // 32 * 32
    wg, wu, wd = rnd(experts, ff, d, dt=bf, scale=0.02), rnd(experts, ff, d, dt=bf, scale=0.02), rnd(experts, d, ff, dt=bf, scale=0.02)
    corr = rnd(experts, scale=0.1)
    for t, name in ((8, "decode"), (4096, "prefill")):
        x = rnd(t, d, dt=bf)
        logits = rnd(t, experts)
        ids, weights = torch.empty(t, top, dtype=torch.int32, device=dev), torch.empty(t, top, device=dev)
        if t > 16:
            big = rnd(1 << 20, experts)
            bi, bw = torch.empty(1 << 20, top, dtype=torch.int32, device=dev), torch.empty(1 << 20, top, device=dev)
            t_new = us(lambda: ops.moe_route_scored(big, top, bi, bw, corr, 4, 2, 1.5))
            t_like = us(lambda: ops.moe_route(big, top, bi, bw))
            entry("moe_route_scored", t_new, t_like, (1 << 20) * (experts * 4 + top * 8), like="moe_route (softmax over the chosen)")
            del big, bi, bw
        ops.moe_route_scored(logits, top, ids, weights, corr, 4, 2, 1.5)
        hbuf = torch.empty(t * top, ff, dtype=bf, device=dev)
        yb = torch.empty(t, d, device=dev)
        slots = torch.zeros(t, dtype=torch.int32, device=dev)
        if t <= 16:
            t_new = us(lambda: (ops.moe_route_scored(logits, top, ids, weights, corr, 4, 2, 1.5),
                                ops.moe_gate_up_pairs(x, wu, None, ids, slots, hbuf, "gelu"), ops.moe_down_pairs(hbuf, wd, ids, weights, slots, yb)))
            t_like = us(lambda: (ops.moe_route(logits, top, ids, weights), ops.moe_gate_up_pairs(x, wg, wu, ids, slots, hbuf, "silu"),
                                 ops.moe_down_pairs(hbuf, wd, ids, weights, slots, yb)))
            touched = min(experts, t * top)
            entry("ungated_experts_" + name, t_new, t_like, nbytes=touched * 2 * ff * d * 2, like_bytes=touched * 3 * ff * d * 2,
                  like="gated experts of the same sizes (pair by pair)")
        else:
            scratch = torch.empty(ops.moe_grouped_scratch_ints(t * top, experts), dtype=torch.int32, device=dev)
            z = torch.empty(t * top, d, device=dev)
            t_new = us(lambda: (ops.moe_route_scored(logits, top, ids, weights, corr, 4, 2, 1.5),
                                ops.moe_grouped(x, wu, None, wd, ids, weights, slots, scratch, hbuf, z, yb, "gelu")), reps=2)
            t_like = us(lambda: (ops.moe_route(logits, top, ids, weights),
                                 ops.moe_grouped(x, wg, wu, wd, ids, weights, slots, scratch, hbuf, z, yb, "silu")), reps=2)
            entry("ungated_experts_" + name, t_new, t_like, flops=4 * t * top * ff * d, like_flops=6 * t * top * ff * d,
                  like="gated experts of the same sizes (sorted tiles)")
    return out


def workload_modadra(a, pk):
    """The Modadra design at the layer sizes of the Qwen2.5 shapes, beside the Fozutar design (the closest one: attention,
    a recurrent mixer and routed experts too) and the dense decoder at the same sizes: decode at the headline batch and
    context, one prompt of `--prefill` tokens, and the new kernels alone."""
    import torch

    from machserve_b200 import ops

    out = {}
    shapes = sorted(SHAPES) if a.modadra_shapes == "all" else [x.strip() for x in a.modadra_shapes.split(",") if x.strip()]
    for shape in shapes:
        raw = SHAPES[shape]
        layers = min(raw["num_hidden_layers"], a.layers or 12)  # (layers of like sizes: twelve tell what all tell)
        res = {"layers": layers}
        steps = max(10, a.steps // 2)
        for which in ("modadra", "fozutar", "dense"):
            kw = {}
            if which != "dense":
                kw = dict(config=(modadra_config if which == "modadra" else fozutar_config)(raw, layers), vocab=raw["vocab_size"])
            b = DecodeBench(a, raw, layers, "bf16", a.batch, a.context + 4 * (steps + a.warmup) + a.batch + 64, **kw)
            times, launches = b.time_decode(a.batch, a.context, steps, a.warmup, blocks=3, sampled=False)
            pms = b.time_prefill(a.prefill, 2, reps=3)
            res[which] = {"decode_ms_per_step": round(times[len(times) // 2], 4), "decode_tokens_per_s": round(a.batch * 1000.0 / times[len(times) // 2], 1),
                          "launches_per_step": launches // steps, "prefill_ms": round(pms, 3), "prefill_tokens_per_s": round(a.prefill * 1000.0 / pms, 1)}
            b.runner.check_device_status()
            b.release_all()
            del b
            free_device_memory()
        if not a.no_points:
            res["kernels"] = time_modadra_kernels(torch, ops, raw, pk)
        free_device_memory()
        out[shape] = res
    return {"batch": a.batch, "context": a.context, "prefill_tokens": a.prefill, "dtype": "bf16",
            "data": "random-init weights drawn on the device, seeded uniform random token ids", "peaks": pk["source"], "sizes": out}


def varolix_config(raw, layers):
    """A Varolix configuration with the layer sizes of the Qwen2 shape `raw`: the same width, vocabulary, feed-forward, heads,
    key heads and head size.  Layers in turns of three: rotary attention (half of every head rotated, waves stretched four
    times past 2,048 positions); normed attention beside a matrix memory of half as many heads of twice the head size in
    their values; latent attention (a latent of four head sizes, a rotated part of half a head size, a query latent of six
    head sizes).  No loop."""
    d, i, v, hq, hkv, hd = sizes(raw)
    att = {"heads": hq, "kv_heads": hkv, "dim": hd, "vdim": hd, "scale": hd ** -0.5,
           "rot": {"dims": hd // 2, "base": 10000.0, "scaling": {"factor": 4.0, "original": 2048, "fast": 32.0, "slow": 1.0}}}
    pair = {"left": {"heads": hq, "kv_heads": hkv, "dim": hd, "vdim": hd, "scale": hd ** -0.5, "q_temp": {"coef": 0.1, "every": 1024}},
            "right": {"heads": max(1, hq // 2), "dim": hd, "vdim": 2 * hd, "gate_cap": 12.0}, "left_scale": 1.0, "right_scale": 0.5}
    lat = {"heads": hq, "dim": hd, "rot_dim": hd // 2, "vdim": hd, "kv_rank": 4 * hd, "q_rank": 6 * hd, "scale": (1.5 * hd) ** -0.5,
           "rot": {"dims": hd // 2, "base": 10000.0}}
    kinds = [("attention", att), ("parallel", pair), ("latent_attention", lat)]
    return {"architecture": "Varolix", "vocab": v, "width": d, "norm": {"eps": 1e-6},
            "layers": [{"type": kinds[n % 3][0], "mixer": kinds[n % 3][1], "mlp": {"kind": "dense", "ff": i}} for n in range(layers)]}


def time_varolix_kernels(torch, ops, raw, pk):
    """The Varolix design's kernels alone, each beside the like kernel of the closest designs at equal sizes where there is
    one (inputs larger than the L2; a CUDA graph of a few launches between events)."""
    d, inter, _, hq, hkv, hd = sizes(raw)
    dev, bf = "cuda:0", torch.bfloat16
    g = torch.Generator(device=dev).manual_seed(0)
    rnd = lambda *shape, dt=torch.float32, scale=1.0: (torch.randn(*shape, device=dev, generator=g) * scale).to(dt)

    def us(fn, reps=5):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            for _ in range(reps):
                fn()
        graph.replay()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        graph.replay()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / reps * 1000

    out = {}

    def entry(name, t_new, t_like=None, nbytes=None, flops=None, like_bytes=None, like_flops=None, like="(no like kernel)"):
        e = {"us": round(t_new, 1), "like": like}
        if t_like is not None:
            e["like_us"] = round(t_like, 1)
        if nbytes:
            e["hbm_frac"] = round(nbytes / t_new / 1e3 / pk["hbm_gbs"], 3)
            if t_like is not None:
                e["like_hbm_frac"] = round((like_bytes or nbytes) / t_like / 1e3 / pk["hbm_gbs"], 3)
        if flops:
            e["tensor_frac"] = round(flops / t_new / 1e6 / pk["bf16_tflops"], 4)
            if t_like is not None:
                e["like_tensor_frac"] = round((like_flops or flops) / t_like / 1e6 / pk["bf16_tflops"], 4)
        out[name] = e

    # the weighted sum of the two mixers' outputs (with the left one's output bias): 32,768 rows
    rows = 32768
    da, db, res = rnd(rows, d), rnd(rows, d), rnd(rows, d)
    w = rnd(d)
    o32, o16 = torch.empty(rows, d, device=dev), torch.empty(rows, d, dtype=bf, device=dev)
    t_new = us(lambda: ops.pair_weighted_sum(da, db, o32, 1.2, 0.9, bias_a=w))
    t_like = us(lambda: ops.norm_pair_mean(da, db, w, w, o32, 1e-6, 0.5))
    entry("pair_weighted_sum", t_new, t_like, rows * d * 12, like="norm_pair_mean (the mean of two normed rows)")
    del da, db, res, o32, o16
    # between the input product and the attention: 16,384 rows
    rows, page = 16384, PAGE
    pos = (torch.arange(rows, dtype=torch.int32, device=dev) % 4096).contiguous()
    slot = (torch.arange(rows, dtype=torch.int32, device=dev) // 4096).contiguous()
    pages = rows // page
    table = torch.arange(pages, dtype=torch.int32, device=dev).view(4, -1).contiguous()
    qkvw = (hq + 2 * hkv) * hd
    proj, bias = rnd(rows, qkvw), rnd(qkvw)
    kp, vp = torch.zeros(pages, hkv, page, hd, dtype=bf, device=dev), torch.zeros(pages, hkv, page, hd, dtype=bf, device=dev)
    qo, qh = torch.empty(rows, hq * hd, device=dev), torch.empty(rows, hq * hd, dtype=bf, device=dev)
    half = torch.zeros(4096, hd // 4, 2, device=dev)
    proj16, qo16 = rnd(rows, qkvw, dt=bf), torch.empty(rows, hq * hd, dtype=bf, device=dev)
    ang = torch.zeros(4096, hd // 2, 2, device=dev)
    t_like = us(lambda: ops.rope_kv_store(proj16, None, pos, slot, table, ang, hd, False, qo16, kp, vp, hq, hkv, hd))
    store_bytes = rows * (qkvw * 4 + hq * hd * 6 + 2 * hkv * hd * 2)
    like_bytes = rows * (qkvw * 2 + hq * hd * 2 + 2 * hkv * hd * 2)
    t_new = us(lambda: ops.rope_store(proj, half, hd // 2, False, pos, slot, table, qo, kp, vp, hq, hkv, hd, hd, q_half=qh, bias=bias))
    entry("rope_store_with_biases", t_new, t_like, store_bytes, like_bytes=like_bytes, like="rope_kv_store (bfloat16 in and out)")
    wn = rnd(hd)
    t_new = us(lambda: ops.head_norm_store(proj, 1e-6, pos, slot, table, qo, kp, vp, hq, hkv, hd, hd, (hq + hkv) * hd, norm=True, wq=wn, wk=wn,
                                           q_half=qh, bias=bias, temp_coef=0.1, temp_every=1024))
    entry("head_norm_store_with_weights_biases_temperature", t_new, t_like, store_bytes, like_bytes=like_bytes,
          like="rope_kv_store (bfloat16 in and out)")
    del proj, proj16, qo, qo16, qh, kp, vp
    # latent attention: norm of the query latent, then rotation, latent norm and the write of the plane
    r, dr, rq = 4 * hd, hd // 2, 6 * hd
    wide = r + dr
    lproj = rnd(rows, rq + wide + hq)
    queries = rnd(rows, hq * (hd + dr))
    lp = torch.zeros(pages, 1, page, wide, dtype=bf, device=dev)
    qw_, qp_ = torch.empty(rows, hq, wide, device=dev), torch.empty(rows, hq, hd, dtype=bf, device=dev)
    wl, wq = rnd(r), rnd(rq)
    tab = torch.zeros(4096, dr // 2, 2, device=dev)
    cq = torch.empty(rows, rq, dtype=bf, device=dev)
    t_new = us(lambda: (ops.gla_output(lproj[:, :rq], None, wq, 1e-6, cq, 1, rq),
                        ops.latent_encode(lproj, rq, wl, 1e-6, tab, dr, pos, slot, table, qw_, qp_, lp, hq, hd, dr, r, queries=queries,
                                          interleaved=False)))
    entry("query_latent_norm_and_latent_encode", t_new, t_like,
          rows * (rq * 6 + hq * (hd + dr) * 4 + wide * 4 + hq * dr * 4 + hq * hd * 2 + wide * 2), like_bytes=like_bytes,
          like="rope_kv_store (bfloat16 in and out)")
    del lproj, queries, qw_, qp_, cq
    # latent attention with a sink over every earlier token (no window): 64 decoding rows at 4,096 tokens and one prompt of 4,096
    ctx, b = 4096, 64
    pages = b * ctx // page
    table = torch.arange(pages, dtype=torch.int32, device=dev).view(b, -1).contiguous()
    lp = rnd(pages, 1, page, wide, dt=bf)
    sk = rnd(hq)
    posd = torch.full((b,), ctx - 1, dtype=torch.int32, device=dev)
    slotd = torch.arange(b, dtype=torch.int32, device=dev)
    if ops.attention_wide_mma_supports(wide, r, wide, False):
        q = rnd(b, hq * wide)
        o = torch.empty(b, hq * r, dtype=bf, device=dev)
        items = b * (-(-hq // 16))
        splits = max(1, min(6 * ops.sm_count() // items, -(-ctx // 64), 32))
        scratch = torch.empty(max(1, ops.attention_wide_mma_scratch_words(items, r, splits)), device=dev)
        t_new = us(lambda: ops.attention_wide_mma(q, lp, lp, o, sk, posd, slotd, table, None, None, b, True, hq, 1, wide, r, None, 0.1, splits,
                                                  scratch))
        entry("latent_sink_attention_decode", t_new, nbytes=b * ctx * wide * 2, like="(no like kernel: one plane read for keys and values)")
        n = ctx
        posp = torch.arange(n, dtype=torch.int32, device=dev)
        slotp = torch.zeros(n, dtype=torch.int32, device=dev)
        qp, op = rnd(n, hq * wide), torch.empty(n, hq * r, dtype=bf, device=dev)
        tile = ops.attention_wide_mma_tile_rows(r)
        u0 = torch.arange(0, n, tile, dtype=torch.int32, device=dev)
        un = torch.full_like(u0, tile)
        t_new = us(lambda: ops.attention_wide_mma(qp, lp, lp, op, sk, posp, slotp, table, u0, un, u0.numel(), False, hq, 1, wide, r, None, 0.1),
                   reps=2)
        entry("latent_sink_attention_prefill", t_new, flops=2 * (n * (n + 1) // 2) * hq * (wide + r),
              like="(no like kernel; multiply-adds of the carried form)")
        del q, o, qp, op
    del lp
    # the matrix memory: gates (4,096 rows), 64 sequences of one token, one sequence of 4,096 tokens, the read-out
    heads, dk, dv, n = max(1, hq // 2), hd, 2 * hd, 4096
    kw, vw = heads * dk, heads * dv
    width = 2 * kw + 2 * vw + 2 * heads
    proj = rnd(n, width, scale=0.3)
    state = torch.zeros(b, ops.mm_state_floats(heads, dk, dv), device=dev)
    gates = torch.empty(n, heads, 4, device=dev)
    bi = rnd(heads)
    cup = torch.tensor([0, n], dtype=torch.int32, device=dev)
    zero = torch.zeros(n, dtype=torch.int32, device=dev)
    cu1 = torch.arange(b + 1, dtype=torch.int32, device=dev)
    i_off, f_off = 2 * kw + 2 * vw, 2 * kw + 2 * vw + heads
    t_new = us(lambda: ops.mm_gates(proj, i_off, f_off, bi, bi, 15.0, state, cup, zero[:1], zero, gates, 1, heads, dk, dv))
    gproj = rnd(n, 2 * kw + 2 * vw + 16, scale=0.1)
    w2 = rnd(kw, 16, dt=bf)
    dec = torch.empty(n, kw, device=dev)
    t_like = us(lambda: ops.gla_decay(gproj[:, 2 * kw + 2 * vw:], w2, None, 16.0, dec))
    entry("mm_gates_one_sequence", t_new, t_like, n * heads * (8 + 16), like_bytes=n * (16 * 4 + kw * 4),
          like="gla_decay (what the gated linear attention computes before its scan)")
    t_new = us(lambda: ops.mm_gates(proj[:b], i_off, f_off, bi, bi, 15.0, state, cu1, slotd, slotd, gates[:b], b, heads, dk, dv))
    entry("mm_gates_decode", t_new, nbytes=b * heads * (8 + 16 + 8))
    og = torch.empty(n, heads, dv + 1, device=dev)
    t_new = us(lambda: ops.mm_scan(proj[:b], 0, kw, 2 * kw, gates[:b], 0.1, state, cu1, slotd, slotd, og[:b], b, heads, dk, dv))
    gstate = torch.zeros(b, heads, dk, dv, device=dev)
    gout = torch.empty(n, vw, device=dev)
    dec.uniform_(0.9, 1.0)
    t_like = us(lambda: ops.gla_scan(gproj[:b], 0, kw, 2 * kw, dec[:b], 0.1, gstate, cu1, slotd, slotd, gout[:b], b, heads, dk, dv))
    entry("mm_scan_decode", t_new, t_like, 2 * b * heads * dk * (dv + 1) * 4, like_bytes=2 * b * heads * dk * dv * 4, like="gla_scan (decode)")
    t_new = us(lambda: ops.mm_scan(proj, 0, kw, 2 * kw, gates, 0.1, state, cup, zero[:1], zero, og, 1, heads, dk, dv, narrow=True), reps=2)
    t_like = us(lambda: ops.gla_scan(gproj, 0, kw, 2 * kw, dec, 0.1, gstate, cup, zero[:1], zero, gout, 1, heads, dk, dv, narrow=True), reps=2)
    # (CUDA-core multiply-adds, the scan is sequential: two products of the state a token in both)
    entry("mm_scan_prefill", t_new, t_like, flops=n * heads * dk * (dv + 1) * 4, like_flops=n * heads * dk * dv * 4, like="gla_scan (one prompt)")
    y = torch.empty(n, vw, dtype=bf, device=dev)
    normw, normd = rnd(vw), rnd(dv)
    t_new = us(lambda: ops.mm_output(og, gates, proj[:, 2 * kw + vw:2 * kw + 2 * vw], normw, 1e-6, y, heads, dv))
    t_like = us(lambda: ops.gla_output(gout, gproj[:, 2 * kw + vw:2 * kw + 2 * vw], normd, 1e-6, y, heads, dv))
    entry("mm_output", t_new, t_like, n * (vw * (4 + 4 + 2) + heads * 20), like_bytes=n * vw * (4 + 4 + 2), like="gla_output")
    return out


def workload_varolix(a, pk):
    """The Varolix design at the layer sizes of the Qwen2.5 shapes, beside the Fozutar design (the closest one: attention
    layers, layers with a matrix state, dense feed-forwards) and the dense decoder at the same sizes: decode at the headline
    batch and context, one prompt of `--prefill` tokens, and the new kernels alone."""
    import torch

    from machserve_b200 import ops

    out = {}
    shapes = sorted(SHAPES) if a.varolix_shapes == "all" else [x.strip() for x in a.varolix_shapes.split(",") if x.strip()]
    for shape in shapes:
        raw = SHAPES[shape]
        layers = min(raw["num_hidden_layers"], a.layers or 12)  # (layers of like sizes: twelve tell what all tell)
        res = {"layers": layers}
        steps = max(10, a.steps // 2)
        for which in ("varolix", "fozutar", "dense"):
            kw = {}
            if which != "dense":
                kw = dict(config=(varolix_config if which == "varolix" else fozutar_config)(raw, layers), vocab=raw["vocab_size"])
            b = DecodeBench(a, raw, layers, "bf16", a.batch, a.context + 4 * (steps + a.warmup) + a.batch + 64, **kw)
            times, launches = b.time_decode(a.batch, a.context, steps, a.warmup, blocks=3, sampled=False)
            pms = b.time_prefill(a.prefill, 2, reps=3)
            res[which] = {"decode_ms_per_step": round(times[len(times) // 2], 4), "decode_tokens_per_s": round(a.batch * 1000.0 / times[len(times) // 2], 1),
                          "launches_per_step": launches // steps, "prefill_ms": round(pms, 3), "prefill_tokens_per_s": round(a.prefill * 1000.0 / pms, 1)}
            b.runner.check_device_status()
            b.release_all()
            del b
            free_device_memory()
        if not a.no_points:
            res["kernels"] = time_varolix_kernels(torch, ops, raw, pk)
        free_device_memory()
        out[shape] = res
    return {"batch": a.batch, "context": a.context, "prefill_tokens": a.prefill, "dtype": "bf16",
            "data": "random-init weights drawn on the device, seeded uniform random token ids", "peaks": pk["source"], "sizes": out}


def workload_serving(a, pk):
    """Qwen2.5-1.5B sizes: 64 requests, prompts of 128 to 2,048 tokens (seeded), 256 new tokens each, through `Engine`
    with its default budget of prompt tokens per step.  All requests arrive at time zero.  Three loads of other prompt
    lengths and token ids run untimed first, as a server that has been up for a while: they load the kernels and
    capture the graphs of the step sizes that keep coming (the timed load's own steps have not been seen before)."""
    import numpy as np
    import torch

    from machserve_b200 import Engine, ModelRunner, SamplingParams
    from machserve_b200.config import config_from_json

    raw = SHAPES["qwen2.5-1.5b"]
    layers = a.layers_serving or raw["num_hidden_layers"]
    cfg = dict(raw)
    cfg["num_hidden_layers"] = layers
    n_req, new, lo, hi, prefill_rows = 64, 256, 128, 2048, 512
    max_seq = hi + new
    runner = ModelRunner.from_random(config_from_json(cfg), seed=0, on_device=True, dtype="bf16", page_size=PAGE,
                                     num_pages=n_req * (-(-max_seq // PAGE)), max_requests=n_req,
                                     max_step_tokens=n_req + prefill_rows, max_seq_len=max_seq)
    wb, kvb = weight_bytes(raw, layers), kv_bytes_per_token(raw, layers)

    def run(seed, lengths_seed=1):
        lengths = [int(x) for x in np.random.default_rng(lengths_seed).integers(lo, hi + 1, size=n_req)]
        eng = Engine(runner=runner, prefill_rows=prefill_rows)
        ids_rng = np.random.default_rng(seed)
        plans = []
        schedule = eng.scheduler.schedule

        def recording():
            plan = schedule()
            plans.append([(e.start, e.count, e.samples) for e in plan.entries])
            return plan

        eng.scheduler.schedule = recording
        prompts = [ids_rng.integers(0, raw["vocab_size"], size=n).tolist() for n in lengths]
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        sids = [eng.add(p, new, params=SamplingParams()) for p in prompts]
        first, steps = {}, 0
        while not eng.all_done():
            out = eng.step()
            steps += 1
            now = time.perf_counter() - t0
            for sid, _ in out:
                if sid not in first:
                    first[sid] = (now, steps)
        torch.cuda.synchronize()
        wall = time.perf_counter() - t0
        made = sum(len(eng.generated(s)) for s in sids)
        for s in sids:
            eng.ack(s)
        return wall, made, first, steps, plans, eng.counters, lengths

    for warm in range(3):
        run(2, 100 + warm)
    wall, made, first, steps, plans, counters, lengths = run(3)
    runner.check_device_status()
    # what the steps as planned have to read and to compute: the slower of the two bounds, step by step
    floor = 0.0
    for plan in plans:
        if not plan:
            continue
        rows = sum(c for _, c, _ in plan)
        keys = sum(c * s + c * (c + 1) // 2 for s, c, _ in plan)
        nbytes = wb + kvb * sum(s + c for s, c, _ in plan)
        flops = step_flops(raw, layers, rows, keys, sum(1 for _, _, w in plan if w))
        floor += max(nbytes / (pk["hbm_gbs"] * 1e9), flops / (pk["bf16_tflops"] * 1e12))
    ttft_ms = sorted(t * 1000 for t, _ in first.values())
    ttft_steps = sorted(s for _, s in first.values())
    p95 = lambda xs: xs[min(len(xs) - 1, int(round(0.95 * (len(xs) - 1))))]
    out = config_block(raw, layers, dtype="bf16", requests=n_req, prompt_tokens_min=lo, prompt_tokens_max=hi,
                       prompt_tokens_total=sum(lengths), new_tokens_each=new, capacity=n_req, prefill_rows=prefill_rows)
    out.update({
        "generated_tokens_per_s": round(made / wall, 1), "prompt_tokens_per_s": round(sum(lengths) / wall, 1),
        "generated_tokens": made, "wall_s": round(wall, 3), "engine_steps": steps, "preemptions": counters["preemptions"],
        "ttft_ms_median": round(statistics.median(ttft_ms), 1), "ttft_ms_p95": round(p95(ttft_ms), 1),
        "ttft_steps_median": statistics.median(ttft_steps), "ttft_steps_p95": p95(ttft_steps),
        "roofline_floor_s": round(floor, 4), "roofline_frac": round(floor / wall, 4),
        "graphs_of_decoding_steps": runner.graph_counts()["decode"], "graphs_of_other_steps": runner.graph_counts()["shapes"],
        "timing": "wall clock around the whole load through Engine.step, host ids in, sampled ids read by the host",
    })
    del runner
    free_device_memory()
    return out


def workload_mixed(a, pk):
    """Qwen2.5-7B sizes: ONE step of eight 512-row portions of 4,096-token prompts (the last portion of each: 3,584
    earlier tokens are in the cache) beside 56 decoding rows at 1,024-token contexts; the step's logits (64 rows)
    are sampled and the tokens read by the host inside the timed region.  Median of the repeats; between repeats
    the eight prompts are given back and brought to 3,584 tokens again."""
    import numpy as np
    import torch

    from machserve_b200 import ModelRunner, SamplingParams, StepEntry
    from machserve_b200.config import config_from_json
    from machserve_b200.sampling.sampler import Sampler

    raw = SHAPES["qwen2.5-7b"]
    layers = a.layers_mixed or raw["num_hidden_layers"]
    cfg = dict(raw)
    cfg["num_hidden_layers"] = layers
    n_dec, ctx, n_pf, prompt, portion, reps = 56, 1024, 8, 4096, 512, 5
    max_seq = prompt + 64
    pages = n_dec * (-(-(ctx + reps + 12) // PAGE)) + n_pf * (-(-prompt // PAGE)) + 8
    runner = ModelRunner.from_random(config_from_json(cfg), seed=0, on_device=True, dtype="bf16", page_size=PAGE,
                                     num_pages=pages, max_requests=n_dec + n_pf,
                                     max_step_tokens=n_pf * portion + n_dec, max_seq_len=max_seq)
    sampler = Sampler(n_dec + n_pf, runner.device)
    rng = np.random.default_rng(4)
    vocab = raw["vocab_size"]
    ids = lambda n: rng.integers(0, vocab, size=n).tolist()
    for at in range(0, n_dec, 4):  # the decoding requests' contexts, four prompts of 1,024 tokens per step
        runner.step([StepEntry(("d", r), ids(ctx), []) for r in range(at, min(at + 4, n_dec))])
    greedy, states = [SamplingParams()] * (n_dec + n_pf), [1] * (n_dec + n_pf)
    times, walls = [], []
    for rep in range(reps + 4):
        for r in range(n_pf):
            runner.release(("p", r))
        for at in range(0, prompt - portion, portion):
            runner.step([StepEntry(("p", r), ids(portion), []) for r in range(n_pf)])
        entries = [StepEntry(("p", r), ids(portion), [portion - 1]) for r in range(n_pf)]
        entries += [StepEntry(("d", r), ids(1), [0]) for r in range(n_dec)]
        torch.cuda.synchronize()
        bracket = a.profile == "mixed" and rep == reps + 3
        if bracket:
            torch.cuda.cudart().cudaProfilerStart()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0 = time.perf_counter()
        e0.record()
        logits = runner.step(entries)
        toks, _ = sampler.sample(logits, greedy, states)
        e1.record()
        torch.cuda.synchronize()
        if bracket:
            torch.cuda.cudart().cudaProfilerStop()
        if rep >= 4:  # the first passes load kernels and size the scratch memory, the second captures the step
            walls.append((time.perf_counter() - t0) * 1000)
            times.append(e0.elapsed_time(e1))
        assert len(toks) == n_dec + n_pf
    runner.check_device_status()
    ms = statistics.median(times)
    rows = n_pf * portion + n_dec
    keys = n_pf * (portion * (prompt - portion) + portion * (portion + 1) // 2) + n_dec * (ctx + (reps + 4) // 2 + 1)
    flops = step_flops(raw, layers, rows, keys, n_dec + n_pf)
    nbytes = weight_bytes(raw, layers) + kv_bytes_per_token(raw, layers) * (n_pf * prompt + n_dec * ctx)
    out = config_block(raw, layers, dtype="bf16", prompt_portions=n_pf, portion_rows=portion, prompt_tokens=prompt,
                       earlier_tokens_in_cache=prompt - portion, decode_rows=n_dec, decode_context=ctx, rows=rows)
    out.update({
        "ms_per_step": round(ms, 3), "ms_min": round(min(times), 3), "ms_max": round(max(times), 3), "repeats": reps,
        "wall_ms_median": round(statistics.median(walls), 3), "rows_per_s": round(rows * 1000.0 / ms, 1),
        "tflops": round(flops / ms / 1e9, 1), "tensor_frac": round(flops / ms / 1e9 / pk["bf16_tflops"], 4),
        "hbm_gbs": round(nbytes / ms / 1e6, 1), "bound": "tensor",
        "timing": "CUDA events around runner.step + sampler + read of the 64 sampled tokens by the host",
    })
    del runner, sampler
    free_device_memory()
    return out


# ------------------------------------------------------------------------------------------------- main


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--context", type=int, default=2048)
    ap.add_argument("--prefill", type=int, default=2048, help="tokens of the timed prompt")
    ap.add_argument("--points", default="1,64", help="further batch sizes for `points` (comma separated)")
    ap.add_argument("--shape", default="qwen2.5-0.5b", choices=sorted(SHAPES), help="layer sizes of the headline")
    ap.add_argument("--model", default=None, help="a model folder (config.json, model.safetensors) instead of a shape")
    ap.add_argument("--layers", type=int, default=None, help="fewer layers than the configuration has (named in config)")
    ap.add_argument("--layers-serving", type=int, default=None, help="the same for the serving_1p5b workload")
    ap.add_argument("--layers-mixed", type=int, default=None, help="the same for the mixed_7b workload")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--dtype", default="bf16", choices=["bf16", "bfloat16", "f32", "fp32", "float32"])
    ap.add_argument("--only", default="headline,fp32,serving_1p5b,mixed_7b",
                    help="which parts to run: headline, fp32, serving_1p5b, mixed_7b (comma separated); venarax, which is not "
                         "among the defaults, times the Venarax design beside the dense decoder at equal layer sizes; fozutar, "
                         "likewise not among the defaults, does the same for the Fozutar design; modadra, not among the defaults "
                         "either, times the Modadra design beside the Fozutar design and the dense decoder; varolix, not among the defaults "
                         "either, does the same for the Varolix design")
    ap.add_argument("--no-points", action="store_true", help="skip the further batch sizes and the prefill (venarax: the kernels alone)")
    ap.add_argument("--venarax-shapes", default="all", help="the shapes of the venarax workload (comma separated), or all")
    ap.add_argument("--fozutar-shapes", default="all", help="the shapes of the fozutar workload (comma separated), or all")
    ap.add_argument("--modadra-shapes", default="all", help="the shapes of the modadra workload (comma separated), or all")
    ap.add_argument("--varolix-shapes", default="all", help="the shapes of the varolix workload (comma separated), or all")
    ap.add_argument("--profile", default=None, choices=["decode", "prefill", "mixed"],
                    help="which timed region is bracketed by cudaProfilerStart/Stop (for ncu --profile-from-start off)")
    ap.add_argument("--kernel", default=None, choices=["attention_prefill", "gemm"],
                    help="time one kernel alone at the configuration's head sizes instead of the step, and print its own line")
    a = ap.parse_args()

    if a.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable":
                          "gqf2008/machserve is Rust + HIP (hiprtc, hipBLAS) for AMD GPUs: no Rust toolchain here, "
                          "no Python package to install, and no CUDA path in its tree"}))
        return 0
    if a.gpus != 1 or int(os.environ.get("WORLD_SIZE", "1")) != 1:
        print(f"bench.py: this engine runs on one GPU; --gpus {a.gpus} is not supported")
        return 2
    a.warmup = max(a.warmup, 3)
    only = {x.strip() for x in a.only.split(",") if x.strip()}
    if a.profile:
        only = {"mixed_7b"} if a.profile == "mixed" else {"headline"}

    import torch

    from machserve_b200 import ops

    pk = peaks()
    if a.kernel == "gemm":
        return time_gemm_pair_tc(torch, ops, a, pk)
    if a.kernel == "attention_prefill":
        return time_attention_prefill(torch, ops, a, pk)
    other = False  # a model folder of another architecture than the dense decoder: bytes are taken from the runner itself
    if a.model:
        raw = json.load(open(os.path.join(a.model, "config.json")))
        other = "num_attention_heads" not in raw
        if not other:
            raw.setdefault("num_key_value_heads", raw["num_attention_heads"])
            raw.setdefault("tie_word_embeddings", False)
        name = os.path.basename(os.path.normpath(a.model))
    else:
        raw, name = SHAPES[a.shape], {"qwen2.5-0.5b": "Qwen2.5-0.5B sizes", "qwen2.5-1.5b": "Qwen2.5-1.5B sizes",
                                      "qwen2.5-7b": "Qwen2.5-7B sizes"}[a.shape]
    full_layers = len(raw["layers"]) if other else raw["num_hidden_layers"]
    layers = full_layers if a.model else (a.layers or full_layers)
    f32 = a.dtype in ("f32", "fp32", "float32")
    elt = 4 if f32 else 2
    points_b = [] if a.no_points else [int(x) for x in a.points.split(",") if x.strip()]

    line = {}
    if "headline" in only:
        max_batch = max([a.batch, *points_b])
        b = DecodeBench(a, raw, layers, a.dtype, max_batch, a.context + 4 * (a.steps + a.warmup) + max_batch + 64, load_dir=a.model,
                        vocab=raw.get("vocab") if other else None)
        if other:  # what a decode step has to read: every weight once, and per live request what each cache group keeps
            held = a.context + a.warmup + a.steps * 3 // 2
            per_request = sum(len(g.runs) * g.need.elements_per_token() * min(held, g.need.window or held) for g in b.runner.cache.groups)
            other_bytes = b.runner.memory_plan()["weights_bytes"] + elt * per_request * a.batch
        clocks = ClockSampler()
        clocks.start()
        times, launches = b.time_decode(a.batch, a.context, a.steps, a.warmup, profile=a.profile == "decode")
        clock_info = clocks.stop()
        ms_step = times[len(times) // 2]
        value = a.batch * 1000.0 / ms_step
        bare, _ = b.time_decode(a.batch, a.context, a.steps, a.warmup, blocks=1, sampled=False)
        e2e = b.time_e2e(a.batch, a.context, a.steps, a.warmup)
        points, points_e2e, prefill = {}, {}, None
        for pb in points_b:
            t, _ = b.time_decode(pb, a.context, a.steps, a.warmup)
            points[f"decode_b{pb}"] = round(pb * 1000.0 / t[len(t) // 2], 1)
            points_e2e[f"decode_b{pb}"] = b.time_e2e(pb, a.context, a.steps, a.warmup)["value"]
        if not a.no_points:
            pms = b.time_prefill(a.prefill, a.warmup, profile=a.profile == "prefill")
            prefill = {"value": round(a.prefill * 1000.0 / pms, 1), "tokens": a.prefill, "ms": round(pms, 3),
                       "frac": None if other else round(prefill_flops(raw, layers, a.prefill) / (pms * 1e-3) / (pk["bf16_tflops"] * 1e12), 4)}
        b.runner.check_device_status()  # raises if a tensor-core kernel gave up one of its bounded waits
        b.release_all()
        del b
        free_device_memory()

        # the median block ran at contexts of about context + warmup + 1.5 * steps tokens
        if other:
            describe = lambda **kw: {"architecture": raw.get("architecture"), "layers": layers, "page_size": PAGE, **kw}
        else:
            describe = lambda **kw: config_block(raw, layers, **kw)
        nbytes = other_bytes if other else decode_bytes(raw, layers, a.batch, a.context + a.warmup + a.steps * 3 // 2, elt)
        achieved = nbytes / (ms_step * 1e-3) / 1e9
        line = {
            "metric": f"decode tokens/s ({name}, batch {a.batch}, {a.context}-token contexts)",
            "value": round(value, 1), "unit": "tokens/s", "n_gpus": 1, "steps": a.steps, "warmup": a.warmup,
            "ms_per_step": round(ms_step, 4), "higher_is_better": True, "scaling": "weak",
            "vs_baseline": round(value / PUBLISHED_DECODE_B8, 2) if a.shape == "qwen2.5-0.5b" and not a.model else None,
            "dtype": "fp32" if f32 else "bf16",
            "data": "synthetic: seeded uniform random token ids, random-init weights N(0, 0.02) drawn on the device",
            "config": describe(
                model=name, global_batch=a.batch, seq_len=a.context, parallelism="single GPU",
                l2="inputs larger than L2 (weights read every step)",
                timed="model + sampler + token copy to host, CUDA events, median of 3 blocks of K steps",
                baseline="reference decode batch 8 on RX 7900 XTX, f32: 626 tok/s", peaks=pk["source"]),
            "spread": {"blocks": len(times), "ms_min": round(times[0], 4), "ms_max": round(times[-1], 4)},
            "logits_only": {"value": round(a.batch * 1000.0 / bare[0], 1), "ms_per_step": round(bare[0], 4),
                            "what": "the model's step alone, no sampler and no copy of tokens"},
            "e2e": e2e, "gpu_launches": launches, "clocks": clock_info,
            "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                         "frac": round(achieved / pk["hbm_gbs"], 4)},
        }
        if prefill:
            line["prefill"] = prefill
        if points:
            line["points"] = points
            line["points_e2e"] = points_e2e
    if "fp32" in only and not f32 and not a.model:
        line["fp32"] = workload_fp32(a, pk, raw, layers)
    if "serving_1p5b" in only:
        line["serving_1p5b"] = workload_serving(a, pk)
    if "mixed_7b" in only:
        line["mixed_7b"] = workload_mixed(a, pk)
    if "venarax" in only:
        line["venarax"] = workload_venarax(a, pk)
    if "fozutar" in only:
        line["fozutar"] = workload_fozutar(a, pk)
    if "modadra" in only:
        line["modadra"] = workload_modadra(a, pk)
    if "varolix" in only:
        line["varolix"] = workload_varolix(a, pk)
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
