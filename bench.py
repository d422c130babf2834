#!/usr/bin/env python3
"""Decode and prefill throughput of the engine on one B200, SmolLM2 shapes, random weights.

    python bench.py --gpus 1 --steps K --warmup W [--model 135m|360m|1.7b] [--batch 8] [--layers L]
    python bench.py --impl reference ...      (prints why the reference cannot run here)

A "step" is one decode step of the whole batch. Method after the reference's ``pp_tg``
(crates/glassbox-bench/src/main.rs:72-96): a prompt in one forward pass, then single-token steps,
warm-up discarded; unlike the reference, decoding is measured at context (the K timed steps end at
the benchmark context length) instead of from an empty cache. Prints ONE JSON line.
"""
import argparse
import gc
import json
import os
import shutil
import subprocess
import sys
import tempfile
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

SHAPES = {  # the three SmolLM2 sizes that Glassbox benchmarks (its README.md:30-34)
    "135m": dict(num_hidden_layers=30, hidden_size=576, num_attention_heads=9, num_key_value_heads=3,
                 intermediate_size=1536, vocab_size=49152, rope_theta=100000.0, rms_norm_eps=1e-5,
                 tie_word_embeddings=True, max_position_embeddings=8192),
    "360m": dict(num_hidden_layers=32, hidden_size=960, num_attention_heads=15, num_key_value_heads=5,
                 intermediate_size=2560, vocab_size=49152, rope_theta=100000.0, rms_norm_eps=1e-5,
                 tie_word_embeddings=True, max_position_embeddings=8192),
    "1.7b": dict(num_hidden_layers=24, hidden_size=2048, num_attention_heads=32, num_key_value_heads=32,
                 intermediate_size=8192, vocab_size=49152, rope_theta=130000.0, rms_norm_eps=1e-5,
                 tie_word_embeddings=True, max_position_embeddings=8192),
}
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            p = json.load(f)
        return {"hbm_gbs": float(p["hbm_gbs"]), "bf16_tflops": float(p["bf16_tflops"]), "source": "measured"}
    except (OSError, KeyError, ValueError, TypeError):
        return dict(FALLBACK_PEAKS)


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons while the timed region runs (read-only)."""
    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
             "clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.rows, self.proc = [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", "0", f"--query-gpu={self.QUERY}",
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        sm = sorted(int(r[0]) for r in self.rows if r and r[0].isdigit())
        mx = [int(r[1]) for r in self.rows if len(r) > 1 and r[1].isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = sorted({n for r in self.rows if len(r) >= 7 for n, v in zip(names, r[3:7]) if v.lower() == "active"})
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": reasons, "samples": len(sm)}


def matrix_params_per_layer(c):
    d, hd = c["hidden_size"], c["hidden_size"] // c["num_attention_heads"]
    qd, kvd, inter = c["num_attention_heads"] * hd, c["num_key_value_heads"] * hd, c["intermediate_size"]
    return d * (qd + 2 * kvd) + qd * d + 2 * inter * d + inter * d


def prefill_flops(c, T):
    """Linear layers 2*params*T, causal attention 2*T^2*qd per layer (QK^T and PV over half the
    square), head on one row."""
    hd = c["hidden_size"] // c["num_attention_heads"]
    qd = c["num_attention_heads"] * hd
    L = c["num_hidden_layers"]
    return L * (2.0 * matrix_params_per_layer(c) * T + 2.0 * T * T * qd) + 2.0 * c["vocab_size"] * c["hidden_size"]


def serving_workload(args):
    """Continuous batching on a mixed workload, after the reference's serving benchmark
    (crates/glassbox-bench/src/main.rs:296-318: random tokens, a spread of prompt and output lengths, a shared
    prefix for some), two requests arriving per step. Wall-clock, host tokens in and sampled tokens out."""
    import numpy as np
    import torch
    import glassbox_b200
    from glassbox_b200 import kernels
    from glassbox_b200.engine.engine import Engine
    from glassbox_b200.engine.scheduler import Request, Scheduler, SchedulerConfig
    from glassbox_b200.models.llama import make_llama_raw_config
    from glassbox_b200.sampling.sampler import SamplerConfig

    model = args.model if args.model != "135m" else "360m"
    shape = dict(SHAPES[model])
    if args.layers:
        shape["num_hidden_layers"] = min(args.layers, shape["num_hidden_layers"])
    n_req, chunk, max_seqs = 64, 512, 64
    rng = np.random.default_rng(1)

    def draw():
        """One workload: fresh tokens every time, so that nothing of an earlier pass is found in the prefix cache."""
        shared = rng.integers(0, shape["vocab_size"], size=384).tolist()
        prompts, outs = [], []
        for i in range(n_req):
            n = int(rng.integers(32, 2049))
            body = rng.integers(0, shape["vocab_size"], size=n).tolist()
            prompts.append(shared + body[384:] if i % 4 == 0 and n > 384 else body)
            outs.append(int(rng.integers(32, 513)))
        return prompts, outs

    tmp = tempfile.mkdtemp(prefix="glassbox_b200_bench_")
    try:
        glassbox_b200.write_random_model(tmp, make_llama_raw_config(**shape), seed=0, store_dtype=torch.bfloat16)
        eng = Engine(tmp, "bfloat16", cache_tokens=n_req * 2600, page_size=16, max_batch_tokens=chunk + max_seqs,
                     max_requests=max_seqs + 2, share_prefixes=True)
        results = {}
        for rep in range(3):          # two passes record graphs; the third, on new tokens, is reported
            prompts, outs = draw()
            sched = Scheduler(eng, SchedulerConfig(token_budget=chunk + max_seqs, max_seqs=max_seqs))
            torch.cuda.synchronize()
            launches0, replays0 = kernels.launch_count, eng.graph_replays
            t0 = time.perf_counter()
            todo = list(zip(prompts, outs))
            while todo or not sched.is_idle():
                for p, n in todo[:2]:     # two arrivals per step: later requests find the shared prefix cached
                    sched.submit(Request(prompt=p, max_tokens=n, sampler=SamplerConfig(temperature=0.8, seed=len(p))))
                del todo[:2]
                sched.step()
            torch.cuda.synchronize()
            dt = time.perf_counter() - t0
            eng.check()
            m = sched.metrics
            results = {"metric": f"serving tok/s, mixed workload (SmolLM2-{model.upper()} shapes)",
                       "value": round(m.generated_tokens / dt, 1), "unit": "generated tokens/s", "n_gpus": 1,
                       "seconds": round(dt, 3), "requests": n_req, "prompt_tokens": m.prompt_tokens,
                       "generated_tokens": m.generated_tokens, "total_tokens_per_s": round((m.prompt_tokens + m.generated_tokens) / dt, 1),
                       "steps": m.steps, "prefix_hit_tokens": m.prefix_hit_tokens, "preemptions": m.preemptions,
                       "graph_replays": eng.graph_replays - replays0, "gpu_launches": kernels.launch_count - launches0,
                       "dtype": "bf16", "data": "synthetic", "impl": "ours",
                       "config": {"model": f"SmolLM2-{model} shapes, random weights", "layers": shape["num_hidden_layers"],
                                  "requests": n_req, "prompt_len": "U(32,2048)", "output_len": "U(32,512)",
                                  "portion": chunk, "max_seqs": max_seqs, "shared_prefix": 384, "page_size": 16,
                                  "arrivals_per_step": 2}}
        print(json.dumps(results))
        return 0
    finally:
        shutil.rmtree(tmp, ignore_errors=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=256)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--model", default="135m", choices=sorted(SHAPES))
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--context", type=int, default=4096)
    ap.add_argument("--layers", type=int, default=0, help="run fewer layers than the configuration has")
    ap.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    ap.add_argument("--no-points", action="store_true", help="skip batch-1/64 decode, prefill and e2e")
    ap.add_argument("--workload", default="decode", choices=["decode", "serving"],
                    help="serving: the mixed workload of the 360M configuration (64 requests, prompts 32-2048, outputs "
                         "32-512, prompt portions of 512, a quarter of the requests sharing a 384-token prefix) through "
                         "the scheduler; prints its own JSON line")
    args = ap.parse_args()

    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable":
                          "RudraSomaiya/glassbox is a CPU-only Rust workspace (no GPU code, no Python package): "
                          "pip cannot install it and there is no cargo/rustc here or on the GPU box"}))
        return 0
    if args.gpus != 1:
        print(f"bench.py: this engine runs on one GPU; --gpus {args.gpus} is not supported")
        return 2

    import numpy as np
    import torch
    import glassbox_b200
    from glassbox_b200 import kernels
    from glassbox_b200.engine.engine import Engine, StepEntry
    from glassbox_b200.engine.scheduler import Request, Scheduler, SchedulerConfig
    from glassbox_b200.models.llama import make_llama_raw_config

    if args.workload == "serving":
        return serving_workload(args)
    K, W, B, CTX = args.steps, max(args.warmup, 3), args.batch, args.context
    shape = dict(SHAPES[args.model])
    full_layers = shape["num_hidden_layers"]
    if args.layers:
        shape["num_hidden_layers"] = min(args.layers, full_layers)
    L = shape["num_hidden_layers"]
    raw = make_llama_raw_config(**shape)
    pk = peaks()
    tmp = tempfile.mkdtemp(prefix="glassbox_b200_bench_")
    try:
        store = torch.bfloat16 if args.dtype == "bfloat16" else torch.float32
        glassbox_b200.write_random_model(tmp, raw, seed=0, store_dtype=store)
        page = 16
        max_b = max(B, 64 if not args.no_points else B)
        pool_tokens = max_b * (CTX + page) + 4096
        eng = Engine(tmp, args.dtype, cache_tokens=pool_tokens, page_size=page, max_batch_tokens=2048,
                     max_requests=max_b + 2)
        rng = np.random.default_rng(0)
        vocab = shape["vocab_size"]

        def prefill(rid, n):
            eng.add_request(rid)
            toks = rng.integers(0, vocab, size=n)
            for i in range(0, n, 2048):
                eng.step([StepEntry(rid, toks[i:i + 2048].tolist(), [])])

        def decode_run(batch, steps, warm):
            """``warm`` untimed then ``steps`` timed decode steps that end at context CTX."""
            start_ctx = max(CTX - steps - warm, 1)
            rids = [f"d{batch}_{i}" for i in range(batch)]
            for r in rids:
                prefill(r, start_ctx)
            nxt = rng.integers(0, vocab, size=(steps + warm, batch))
            zeros = ([0.0] * batch, [0.0] * batch)

            def one(s):
                eng.step([StepEntry(r, [int(nxt[s, i])], [0]) for i, r in enumerate(rids)], sampling=zeros)
            for s in range(warm):
                one(s)
            torch.cuda.synchronize()
            launches0 = kernels.launch_count
            print(f"decode batch {batch}: {launches0} kernel launches before the timed steps (for ncu -s)", file=sys.stderr)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for s in range(warm, warm + steps):
                one(s)
            e1.record()
            torch.cuda.synchronize()
            ms = e0.elapsed_time(e1)
            eng.check()
            for r in rids:
                eng.free_request(r)
            mean_ctx = start_ctx + warm + steps / 2.0
            return ms, kernels.launch_count - launches0, mean_ctx

        clocks = ClockSampler()
        clocks.start()
        ms, launches, mean_ctx = decode_run(B, K, W)
        clock_info = clocks.stop()
        ms_per_step = ms / K
        value = B * K / (ms / 1e3)
        weight_bytes = eng.weight_bytes()
        kv_bytes = B * mean_ctx * eng.cache_bytes_per_token()
        achieved = (weight_bytes + kv_bytes) / (ms_per_step / 1e3) / 1e9

        out = {
            "metric": f"decode tok/s at batch {args.batch} (SmolLM2-{args.model.upper()} shapes); prefill tok/s at 2,048 tokens",
            "value": round(value, 1), "unit": "tokens/s", "n_gpus": 1, "steps": K, "warmup": W,
            "ms_per_step": round(ms_per_step, 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "bf16" if args.dtype == "bfloat16" else "fp32", "data": "synthetic", "impl": "ours",
            "config": {"model": f"SmolLM2-{args.model} shapes, random weights", "global_batch": B, "seq_len": CTX,
                       "parallelism": "single GPU", "layers": L, "layers_in_config": full_layers,
                       "hidden": shape["hidden_size"], "heads": shape["num_attention_heads"],
                       "kv_heads": shape["num_key_value_heads"], "head_dim": shape["hidden_size"] // shape["num_attention_heads"],
                       "intermediate": shape["intermediate_size"], "vocab": vocab, "rope_theta": shape["rope_theta"],
                       "tied_head": shape["tie_word_embeddings"], "page_size": page,
                       "decode_ctx_start": int(mean_ctx - K / 2.0), "decode_ctx_end": int(mean_ctx + K / 2.0),
                       "l2": "inputs>L2 (weights+KV per step exceed 126 MB)", "cuda_graph": eng.use_graphs},
            "clocks": clock_info,
            "gpu_launches": int(launches),
            "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                         "frac": round(achieved / pk["hbm_gbs"], 4), "peak_source": pk["source"],
                         "bytes_per_step": int(weight_bytes + kv_bytes)},
        }

        if not args.no_points:
            points = {}
            for b in (1, 64):
                steps_b = max(32, min(K, 128))
                m, _, _ = decode_run(b, steps_b, W)
                points[f"decode_b{b}"] = round(b * steps_b / (m / 1e3), 1)
            out["points"] = points

            # prefill of 2,048 tokens in one step
            T = 2048
            toks = rng.integers(0, vocab, size=T).tolist()
            times = []
            for rep in range(8):
                eng.add_request("p")
                torch.cuda.synchronize()
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                eng.step([StepEntry("p", toks, [T - 1])])
                e1.record()
                torch.cuda.synchronize()
                eng.free_request("p")
                if rep >= 3:     # three warm-up repetitions (the second one records the step's CUDA graph)
                    times.append(e0.elapsed_time(e1))
            pms = sum(times) / len(times)
            flops = prefill_flops(shape, T)
            out["prefill"] = {"value": round(T / (pms / 1e3), 1), "tokens": T, "ms": round(pms, 3),
                              "frac": round(flops / (pms / 1e3) / (pk["bf16_tflops"] * 1e12), 4),
                              "peak_tflops": pk["bf16_tflops"], "peak_source": pk["source"]}

            # end to end through the scheduler: host tokens in, sampled tokens out, every step
            sched = Scheduler(eng, SchedulerConfig(token_budget=2048, max_seqs=B))
            e2e_steps = max(32, min(K, 256))
            # Requests that finish their prompts early decode a few tokens while the others still prefill; leave
            # room for that, so that every request is still live (and within the context) at the last timed step:
            # a batch that shrinks changes the step's shape, and recording a new CUDA graph is not a decode step.
            early = 2 * (-(-B * CTX // 2048))
            start_ctx = max(CTX - e2e_steps - W - 1 - early, 1)
            for i in range(B):
                sched.submit(Request(prompt=rng.integers(0, vocab, size=start_ctx).tolist(),
                                     max_tokens=e2e_steps + W + 1 + early))
            while any(s.generated == 0 for s in sched.running) or sched.waiting:
                sched.step()
            for _ in range(W):
                sched.step()
            torch.cuda.synchronize()
            gc.collect()
            gc.freeze()      # the model's long-lived objects leave the collector's view: no full collection mid-run
            made = sum(s.generated for s in sched.running)
            t0 = time.perf_counter()
            h2d = 0
            step_s = []
            for _ in range(e2e_steps):
                ts = time.perf_counter()
                sched.step()
                step_s.append(time.perf_counter() - ts)
                h2d += eng.h2d_bytes_last
            torch.cuda.synchronize()
            dt = time.perf_counter() - t0
            gc.unfreeze()
            made = sum(s.generated for s in sched.running) - made
            assert len(sched.running) == B and made == B * e2e_steps, "a request ended inside the timed region"
            slow = sorted(range(e2e_steps), key=lambda i: -step_s[i])[:3]
            print("e2e: slowest steps (index, ms): " + ", ".join(f"{i}: {step_s[i] * 1e3:.1f}" for i in slow)
                  + f"; median {sorted(step_s)[e2e_steps // 2] * 1e3:.3f} ms", file=sys.stderr)
            out["e2e"] = {"value": round(made / dt, 1), "unit": "tokens/s", "steps": e2e_steps,
                          "h2d_bytes_per_step": int(h2d / e2e_steps), "d2h_bytes_per_step": 4 * B,
                          "api": "Scheduler.submit/step (host token ids in, sampled ids out)"}
            sched.run_until_idle()
        print(json.dumps(out))
        return 0
    finally:
        shutil.rmtree(tmp, ignore_errors=True)


if __name__ == "__main__":
    sys.exit(main())
