#!/usr/bin/env python3
"""Decode and prefill throughput of the engine on one B200, SmolLM2 shapes, random weights.

    python bench.py --gpus 1 --steps K --warmup W [--model 135m|360m|1.7b] [--batch 8] [--layers L]
    python bench.py --impl reference ...      (prints why the reference cannot run here)

A "step" is one decode step of the whole batch. Method after the reference's ``pp_tg``
(crates/glassbox-bench/src/main.rs:72-96): a prompt in one forward pass, then single-token steps,
warm-up discarded, mean and standard deviation over repetitions; unlike the reference, decoding is
measured at context (the K timed steps end at the benchmark context length) instead of from an empty
cache. Prints ONE JSON line.

The line's ``value`` is the named model's decode rate at ``--batch`` over exactly K timed steps. Beside it:
``points`` (decode at batch 1 and 64 and, unless ``--no-others``, the other two SmolLM2 sizes at batch 1/8/64
with their prefill, the 360M serving workload, and the true 32-bit path at 135M), ``points_frac`` (each
point's fraction of its roofline: HBM for decoding, bf16 tensor peak for prefill), ``stats`` (mean and
standard deviation of the repeated regions), ``prefill``, ``roofline``, ``e2e`` and ``cpu_baseline`` (the plain
C++ float32 implementation under tests/plain on this machine's CPU, timed the reference's way).
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

    def __init__(self, gpu: str = "0"):
        """``gpu``: what ``nvidia-smi -i`` takes: the UUID of the device the benchmark runs on (index 0 of this
        process need not be index 0 of the machine)."""
        self.rows, self.proc, self.gpu = [], None, gpu

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", self.gpu, f"--query-gpu={self.QUERY}",
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
                "reasons": reasons, "samples": len(sm), "gpu": self.gpu}


def device_uuid() -> str:
    """The UUID of cuda:0 of this process in nvidia-smi's spelling, or "0" if torch does not tell."""
    import torch
    try:
        u = str(torch.cuda.get_device_properties(0).uuid)
        return u if u.startswith("GPU-") else "GPU-" + u
    except Exception:
        return "0"


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


def mean_sd(xs):
    m = sum(xs) / len(xs)
    return m, (sum((x - m) ** 2 for x in xs) / max(len(xs) - 1, 1)) ** 0.5


class ModelBench:
    """One SmolLM2 size with random weights in an engine, and the timed regions on it."""

    def __init__(self, model: str, dtype: str, max_batch: int, ctx: int, layers: int = 0, seed: int = 0):
        import numpy as np
        import torch
        import glassbox_b200
        from glassbox_b200.engine.engine import Engine
        from glassbox_b200.models.llama import make_llama_raw_config
        self.model, self.dtype, self.ctx = model, dtype, ctx
        self.shape = dict(SHAPES[model])
        self.full_layers = self.shape["num_hidden_layers"]
        if layers:
            self.shape["num_hidden_layers"] = min(layers, self.full_layers)
        self.tmp = tempfile.mkdtemp(prefix="glassbox_b200_bench_")
        store = torch.bfloat16 if dtype == "bfloat16" else torch.float32
        glassbox_b200.write_random_model(self.tmp, make_llama_raw_config(**self.shape), seed=seed, store_dtype=store)
        self.page = 16
        self.eng = Engine(self.tmp, dtype, cache_tokens=max_batch * (ctx + self.page) + 4096, page_size=self.page,
                          max_batch_tokens=2048, max_requests=max_batch + 2)
        self.rng = np.random.default_rng(seed)
        self.vocab = self.shape["vocab_size"]

    def close(self):
        import torch
        self.eng = None
        shutil.rmtree(self.tmp, ignore_errors=True)
        gc.collect()
        torch.cuda.empty_cache()

    def _prefill(self, rid, n):
        from glassbox_b200.engine.engine import StepEntry
        self.eng.add_request(rid)
        toks = self.rng.integers(0, self.vocab, size=n)
        for i in range(0, n, 2048):
            self.eng.step([StepEntry(rid, toks[i:i + 2048].tolist(), [])])

    def decode(self, batch: int, steps: int, warm: int, reps: int = 1):
        """``warm`` untimed steps, then ``reps`` timed regions of ``steps`` decode steps each, the last of which ends at
        the context length. Returns (ms of each region, kernel launches of the first region, mean context of the timed steps)."""
        import torch
        from glassbox_b200 import kernels
        from glassbox_b200.engine.engine import StepEntry
        eng = self.eng
        total = warm + reps * steps
        start_ctx = max(self.ctx - total, 1)
        rids = [f"d{batch}_{i}" for i in range(batch)]
        for r in rids:
            self._prefill(r, start_ctx)
        nxt = self.rng.integers(0, self.vocab, size=(total, batch))
        zeros = [1] * batch          # every row sampled on the device from its request's state (greedy: no state was set)

        def one(s):
            eng.step([StepEntry(r, [int(nxt[s, i])], [0]) for i, r in enumerate(rids)], sampling=zeros)
        for s in range(warm):
            one(s)
        torch.cuda.synchronize()
        regions, launches = [], None
        for rep in range(reps):
            before = kernels.launch_count
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for s in range(warm + rep * steps, warm + (rep + 1) * steps):
                one(s)
            e1.record()
            torch.cuda.synchronize()
            regions.append(e0.elapsed_time(e1))
            launches = launches if launches is not None else kernels.launch_count - before
        eng.check()
        for r in rids:
            eng.free_request(r)
        return regions, launches, start_ctx + warm + reps * steps / 2.0

    def decode_bytes(self, batch: int, mean_ctx: float) -> float:
        """What a decode step has to read: every weight once, and the cache of the live requests."""
        return self.eng.weight_bytes() + batch * mean_ctx * self.eng.cache_bytes_per_token()

    def prefill(self, T: int = 2048, reps: int = 5):
        """ms of each of ``reps`` single-step prefills of T tokens, after three warm-up repetitions (the second records
        the step's CUDA graph)."""
        import torch
        from glassbox_b200.engine.engine import StepEntry
        toks = self.rng.integers(0, self.vocab, size=T).tolist()
        times = []
        for rep in range(reps + 3):
            self.eng.add_request("p")
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            self.eng.step([StepEntry("p", toks, [T - 1])])
            e1.record()
            torch.cuda.synchronize()
            self.eng.free_request("p")
            if rep >= 3:
                times.append(e0.elapsed_time(e1))
        return times

    def end_to_end(self, batch: int, steps: int, warm: int):
        """Decode tokens a second through ``Scheduler.submit`` / ``step``: host token ids in, sampled ids out, every step."""
        import torch
        from glassbox_b200.engine.scheduler import Request, Scheduler, SchedulerConfig
        eng = self.eng
        sched = Scheduler(eng, SchedulerConfig(token_budget=2048, max_seqs=batch))
        # Requests that finish their prompts early decode a few tokens while the others still prefill; leave room for
        # that, so that every request is still live (and within the context) at the last timed step: a batch that
        # shrinks changes the step's shape, and recording a new CUDA graph is not a decode step.
        early = 2 * (-(-batch * self.ctx // 2048))
        start_ctx = max(self.ctx - steps - warm - 1 - early, 1)
        for i in range(batch):
            sched.submit(Request(prompt=self.rng.integers(0, self.vocab, size=start_ctx).tolist(),
                                 max_tokens=steps + warm + 1 + early))
        while any(s.generated == 0 for s in sched.running) or sched.waiting:
            sched.step()
        for _ in range(warm):
            sched.step()
        torch.cuda.synchronize()
        gc.collect()
        gc.freeze()      # the model's long-lived objects leave the collector's view: no full collection mid-run
        made = sum(s.generated for s in sched.running)
        t0 = time.perf_counter()
        h2d, step_s = 0, []
        for _ in range(steps):
            ts = time.perf_counter()
            sched.step()
            step_s.append(time.perf_counter() - ts)
            h2d += eng.h2d_bytes_last
        torch.cuda.synchronize()
        dt = time.perf_counter() - t0
        gc.unfreeze()
        made = sum(s.generated for s in sched.running) - made
        assert len(sched.running) == batch and made == batch * steps, "a request ended inside the timed region"
        slow = sorted(range(steps), key=lambda i: -step_s[i])[:3]
        print("e2e: slowest steps (index, ms): " + ", ".join(f"{i}: {step_s[i] * 1e3:.1f}" for i in slow)
              + f"; median {sorted(step_s)[steps // 2] * 1e3:.3f} ms", file=sys.stderr)
        sched.run_until_idle()
        return {"value": round(made / dt, 1), "unit": "tokens/s", "steps": steps, "h2d_bytes_per_step": int(h2d / steps),
                "d2h_bytes_per_step": 4 * batch, "median_step_ms": round(sorted(step_s)[steps // 2] * 1e3, 4),
                "api": "Scheduler.submit/step (host token ids in, sampled ids out)"}


def cpu_baseline(folder: str):
    """The plain C++ float32 implementation (tests/plain/ref_forward.cpp: sequential dot products, a contiguous cache,
    four threads) on this machine's CPU, timed as the reference times itself: a 512-token prompt in one pass, then 128
    tokens one at a time from an empty cache."""
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    try:
        from plain.ref_forward import pp_tg
        pp, tg = pp_tg(folder, 512, 128, reps=1)
        return {"pp512_tok_s": round(pp, 1), "tg128_tok_s": round(tg, 1), "threads": int(os.environ.get("REF_THREADS", "4")),
                "what": "tests/plain/ref_forward.cpp, float32, this machine's CPU"}
    except Exception as e:          # no C++ compiler on the machine: the baseline is context, not the measurement
        return {"unavailable": f"{type(e).__name__}: {e}"[:200]}


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
    eng = None
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
        return results
    finally:
        eng = None
        shutil.rmtree(tmp, ignore_errors=True)
        gc.collect()
        torch.cuda.empty_cache()


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
    ap.add_argument("--no-points", action="store_true", help="only the headline region: no other batches, prefill or e2e")
    ap.add_argument("--no-others", action="store_true",
                    help="skip the other model sizes, the serving workload, the 32-bit path and the CPU baseline")
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

    import torch  # noqa: F401
    if args.workload == "serving":
        print(json.dumps(serving_workload(args)))
        return 0
    K, W, B, CTX = args.steps, max(args.warmup, 3), args.batch, args.context
    pk = peaks()
    hbm, tflops = pk["hbm_gbs"], pk["bf16_tflops"]
    REPS = 3
    points, frac, stats = {}, {}, {}

    mb = ModelBench(args.model, args.dtype, max(B, 64 if not args.no_points else B), CTX, args.layers)
    try:
        shape = mb.shape
        clocks = ClockSampler(device_uuid())
        clocks.start()
        regions, launches, mean_ctx = mb.decode(B, K, W, reps=1)          # the headline: exactly K timed steps
        clock_info = clocks.stop()
        ms = regions[0]
        ms_per_step = ms / K
        value = B * K / (ms / 1e3)
        step_bytes = mb.decode_bytes(B, mean_ctx)
        achieved = step_bytes / (ms_per_step / 1e3) / 1e9
        out = {
            "metric": f"decode tok/s at batch {B} (SmolLM2-{args.model.upper()} shapes); prefill tok/s at 2,048 tokens",
            "value": round(value, 1), "unit": "tokens/s", "n_gpus": 1, "steps": K, "warmup": W,
            "ms_per_step": round(ms_per_step, 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "bf16" if args.dtype == "bfloat16" else "fp32", "data": "synthetic", "impl": "ours",
            "config": {"model": f"SmolLM2-{args.model} shapes, random weights", "global_batch": B, "seq_len": CTX,
                       "parallelism": "single GPU", "layers": shape["num_hidden_layers"], "layers_in_config": mb.full_layers,
                       "hidden": shape["hidden_size"], "heads": shape["num_attention_heads"],
                       "kv_heads": shape["num_key_value_heads"], "head_dim": shape["hidden_size"] // shape["num_attention_heads"],
                       "intermediate": shape["intermediate_size"], "vocab": shape["vocab_size"], "rope_theta": shape["rope_theta"],
                       "tied_head": shape["tie_word_embeddings"], "page_size": mb.page,
                       "decode_ctx_start": int(mean_ctx - K / 2.0), "decode_ctx_end": int(mean_ctx + K / 2.0),
                       "l2": "inputs>L2 (weights+KV per step exceed 126 MB)", "cuda_graph": mb.eng.use_graphs},
            "clocks": clock_info,
            "gpu_launches": int(launches),
            "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": hbm, "unit": "GB/s",
                         "frac": round(achieved / hbm, 4), "peak_source": pk["source"], "bytes_per_step": int(step_bytes)},
        }

        def decode_point(bench, name, b, steps):
            """Three timed regions of ``steps`` steps at batch ``b``: tokens/s of the mean, with its roofline fraction."""
            regs, _, ctx_mean = bench.decode(b, steps, W, reps=REPS)
            per = [r / steps for r in regs]
            m, sd = mean_sd(per)
            points[name] = round(b / (m / 1e3), 1)
            frac[name] = round(bench.decode_bytes(b, ctx_mean) / (m / 1e3) / 1e9 / hbm, 4)
            stats[name] = {"ms_per_step": round(m, 4), "sd": round(sd, 4), "reps": REPS, "steps": steps}

        def prefill_point(bench, name):
            times = bench.prefill(2048)
            m, sd = mean_sd(times)
            fl = prefill_flops(bench.shape, 2048) / (m / 1e3) / (tflops * 1e12)
            points[name] = round(2048 / (m / 1e3), 1)
            frac[name] = round(fl, 4)
            stats[name] = {"ms": round(m, 3), "sd": round(sd, 3), "reps": len(times)}
            return m, fl

        if not args.no_points:
            steps_b = max(32, min(K, 64))
            decode_point(mb, f"decode_b{B}_repeated", B, steps_b)
            for b in (1, 64):
                decode_point(mb, f"decode_b{b}", b, steps_b)
            pms, pfrac = prefill_point(mb, "prefill_2048")
            out["prefill"] = {"value": points.pop("prefill_2048"), "tokens": 2048, "ms": round(pms, 3), "frac": round(pfrac, 4),
                              "peak_tflops": tflops, "peak_source": pk["source"], "sd_ms": stats["prefill_2048"]["sd"]}
            frac.pop("prefill_2048")
            out["e2e"] = mb.end_to_end(B, max(32, min(K, 256)), W)
            if not args.no_others and args.dtype == "bfloat16":
                out["cpu_baseline"] = cpu_baseline(mb.tmp)
    finally:
        mb.close()

    if not args.no_points and not args.no_others and args.dtype == "bfloat16":
        layers_note = {}
        for other in [m for m in ("135m", "360m", "1.7b") if m != args.model]:
            ob = ModelBench(other, "bfloat16", 64, CTX)
            try:
                for b in (1, 8, 64):
                    decode_point(ob, f"{other}_decode_b{b}", b, 32)
                prefill_point(ob, f"{other}_prefill_2048")
                layers_note[other] = f"{ob.shape['num_hidden_layers']} of {ob.full_layers} layers"
            finally:
                ob.close()
        fb = ModelBench(args.model, "float32", B, CTX)          # the true 32-bit path: FMA products, float32 cache
        try:
            regs, _, _ = fb.decode(B, 16, W, reps=REPS)
            m, sd = mean_sd([r / 16 for r in regs])
            times = fb.prefill(2048, reps=3)
            pm, psd = mean_sd(times)
            out["points_fp32"] = {f"decode_b{B}": round(B / (m / 1e3), 1), "decode_ms_per_step": round(m, 4), "decode_sd": round(sd, 4),
                                  "prefill_2048": round(2048 / (pm / 1e3), 1), "prefill_ms": round(pm, 3), "prefill_sd": round(psd, 3)}
        finally:
            fb.close()
        srv = serving_workload(argparse.Namespace(model="360m", layers=0))
        points["360m_serving_generated_tok_s"] = srv["value"]
        points["360m_serving_total_tok_s"] = srv["total_tokens_per_s"]
        out["serving"] = {k: srv[k] for k in ("seconds", "requests", "prompt_tokens", "generated_tokens", "steps",
                                               "prefix_hit_tokens", "preemptions", "graph_replays")}
        out["points_layers"] = layers_note
    if points:
        out["points"] = points
        out["points_frac"] = frac
        out["stats"] = stats
    print(json.dumps(out))
    return 0


if __name__ == "__main__":
    sys.exit(main())
