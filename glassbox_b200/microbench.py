"""Times single kernels on SmolLM2 shapes with CUDA events, inside a CUDA graph (no launch overhead),
over operands that rotate through more memory than L2 holds.

    python -m glassbox_b200.microbench gemm_stream [135m|360m|1.7b ...]   weight-streaming GEMM, 1..64 rows
    python -m glassbox_b200.microbench gemm_tc                           tcgen05 GEMM against torch.matmul
    python -m glassbox_b200.microbench attention_decode [batch ...]      paged decode attention at context 4096
    python -m glassbox_b200.microbench attention_splits HEADS KV_HEADS BATCH [CONTEXT]
                                                                         the large-batch decode attention at 1 to 6 splits
    python -m glassbox_b200.microbench attention_prefill                 flash attention, one 2048-token prompt
    python -m glassbox_b200.microbench float32                           the 32-bit path's kernels: FMA GEMM, decode and rows attention
    python -m glassbox_b200.microbench small                             embedding, RMSNorm, rotation + cache write, SwiGLU, sampling
    python -m glassbox_b200.microbench decode_program [batch ...]        a decode step as a kernel chain and as a persistent kernel
    python -m glassbox_b200.microbench layer_gemms [rows ...]            the four products of a decode layer as the layer runs them

Prints one line per case: microseconds and GB/s or TFLOP/s of the algorithmic bytes or flops. With ``--once`` after
the case's name every kernel is launched exactly once and nothing is timed: the form in which a profiler captures one
launch of each kernel.
"""
from __future__ import annotations

import sys

import torch

from . import kernels

DEV = "cuda:0"
L2_BYTES = 126e6

#: (name, output rows N, K, gated) of the per-layer matrices and the head
FAMILIES = {
    "135m": [("qkv", 960, 576, False), ("o", 576, 576, False), ("gate_up", 1536, 576, True), ("down", 576, 1536, False),
             ("head", 49152, 576, False)],
    "360m": [("qkv", 1600, 960, False), ("o", 960, 960, False), ("gate_up", 2560, 960, True), ("down", 960, 2560, False),
             ("head", 49152, 960, False)],
    "1.7b": [("qkv", 6144, 2048, False), ("o", 2048, 2048, False), ("gate_up", 8192, 2048, True),
             ("down", 2048, 8192, False), ("head", 49152, 2048, False)],
}


ONCE = False


def graph_time(fn, reps: int = 12, outer: int = 5) -> float:
    """Mean microseconds of one ``fn()`` among ``reps`` captured in a graph that is replayed ``outer`` times."""
    fn()
    torch.cuda.synchronize()
    if ONCE:
        return float("nan")
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        for _ in range(reps):
            fn()
    for _ in range(3):
        g.replay()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(outer):
        g.replay()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) * 1e3 / (reps * outer)


def _rotating(rows: int, k: int):
    """Enough copies of a [rows, k] bfloat16 matrix that consecutive calls never find theirs in L2."""
    n = max(2, min(12, int(3 * L2_BYTES / (rows * k * 2)) + 1))
    return [(torch.randn(rows, k, device=DEV) * 0.05).bfloat16() for _ in range(n)]


def bench_gemm_stream(families) -> None:
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    for fam in families or list(FAMILIES):
        for name, n, k, gated in FAMILIES[fam]:
            rows = 2 * n if gated else n
            ws = _rotating(rows, k)
            for m in (1, 8, 16, 32, 64):
                a = torch.randn(m, k, device=DEV).bfloat16()
                c = torch.empty(m, n, device=DEV, dtype=torch.bfloat16 if gated else torch.float32)
                turn = [0]

                def stream():
                    kernels.gemm_stream(a, ws[turn[0] % len(ws)], c, gated=gated)
                    turn[0] += 1

                def tiles():
                    w = ws[turn[0] % len(ws)]
                    kernels.gemm_tc_gated(a, w, c, status) if gated else kernels.gemm_tc(a, w, c, False, status)
                    turn[0] += 1

                t = graph_time(stream)
                line = f"{fam} {name:8s} {rows:6d} x {k:5d} rows {m:3d}: stream {t:7.1f} us {rows * k * 2 / t / 1e3:6.0f} GB/s"
                if m >= 16 and kernels.gemm_tc_supported(a, ws[0], c):
                    line += f" | tcgen05 {graph_time(tiles):7.1f} us"
                print(line, flush=True)
    kernels.check_status(status)


def bench_gemm_tc() -> None:
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    for name, m, n, k in [("135m qkv", 2048, 960, 576), ("135m o", 2048, 576, 576), ("135m gate_up", 2048, 3072, 576),
                          ("135m down", 2048, 576, 1536), ("360m qkv", 2048, 1600, 960), ("360m o", 2048, 960, 960),
                          ("360m gate_up", 2048, 5120, 960), ("360m down", 2048, 960, 2560),
                          ("1.7b qkv", 2048, 6144, 2048), ("1.7b gate_up", 2048, 16384, 2048),
                          ("1.7b down", 2048, 2048, 8192), ("square", 8192, 8192, 8192)]:
        a = torch.randn(m, k, device=DEV).bfloat16()
        w = torch.randn(n, k, device=DEV).bfloat16()
        c = torch.empty(m, n, device=DEV).bfloat16()
        t = graph_time(lambda: kernels.gemm_tc(a, w, c, False, status), reps=6)
        t2 = graph_time(lambda: torch.matmul(a, w.T, out=c), reps=6)
        fl = 2.0 * m * n * k
        print(f"{name:13s} {m} x {n} x {k}: tcgen05 {t:8.1f} us {fl / t / 1e6:7.1f} TFLOP/s | torch.matmul {t2:8.1f} us "
              f"{fl / t2 / 1e6:7.1f} TFLOP/s", flush=True)
    kernels.check_status(status)


def bench_attention_decode(batches, nh: int = 9, nkv: int = 3, ctx: int = 4096, sweep: bool = False) -> None:
    """The planner's variant for each batch; with ``sweep`` the four-warp, 16-key variant at 1 to 6 splits as well."""
    hd, ps = 64, 16
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    for m in batches or (1, 8, 64):
        per = ctx // ps
        kc = torch.randn(m * per + 4, nkv, ps, hd, device=DEV).bfloat16()
        vc = torch.randn_like(kc)
        tables = torch.arange(m * per, dtype=torch.int32, device=DEV).view(m, per).contiguous()
        row_seq = torch.arange(m, dtype=torch.int32, device=DEV)
        pos = torch.full((m,), ctx - 1, dtype=torch.int32, device=DEV)
        q = torch.randn(m, nh * hd, device=DEV).bfloat16()
        o = torch.empty_like(q)
        plans = [kernels.decode_mma_plan(m, nkv, hd, ctx)] + ([(s, 16, 4) for s in range(1, 7)] if sweep else [])
        for splits, block_keys, warps in plans:
            pa = torch.empty(m * nh * warps * splits * hd, device=DEV)
            pm = torch.empty(m * nh * warps * splits * 2, device=DEV)
            cn = torch.zeros(m * nkv, dtype=torch.int32, device=DEV)
            t = graph_time(lambda: kernels.attention_decode_mma(q, o, kc, vc, tables, row_seq, pos, nh, nkv, hd, ps, hd ** -0.5,
                                                                None, splits, pa, pm, cn, status, block_keys, warps))
            nbytes = m * ctx * nkv * hd * 2 * 2
            print(f"attention_decode_mma heads {nh}/{nkv} batch {m:3d} ctx {ctx} splits {splits} keys/iteration {block_keys or 32} "
                  f"warps {warps}: {t:7.1f} us {nbytes / t / 1e3:6.0f} GB/s", flush=True)
    kernels.check_status(status)


def bench_attention_prefill() -> None:
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    for nh, nkv, hd, t_len, ps in [(9, 3, 64, 2048, 16), (15, 5, 64, 2048, 16), (32, 32, 64, 2048, 16), (32, 32, 64, 8192, 16),
                                   (32, 32, 64, 8192, 128)]:
        per = t_len // ps
        kc = torch.randn(per + 2, nkv, ps, hd, device=DEV).bfloat16()
        vc = torch.randn_like(kc)
        tables = torch.arange(per, dtype=torch.int32, device=DEV).view(1, per).contiguous()
        first = torch.tensor([0, t_len], dtype=torch.int32, device=DEV)
        start = torch.zeros(1, dtype=torch.int32, device=DEV)
        q = torch.randn(t_len, nh * hd, device=DEV).bfloat16()
        o = torch.empty_like(q)
        fl = 2.0 * t_len * t_len * nh * hd   # QK^T and PV over the causal half
        for name, fn in (("mma.sync", kernels.attention_prefill), ("tcgen05", kernels.attention_prefill_tc)):
            t = graph_time(lambda: fn(q, o, kc, vc, tables, first, start, t_len, nh, nkv, hd, ps, hd ** -0.5, None, status),
                           reps=6)
            print(f"attention_prefill {name:8s} heads {nh}/{nkv} x {hd}, {t_len} tokens, page {ps}: {t:7.1f} us {fl / t / 1e6:6.1f} TFLOP/s",
                  flush=True)
    kernels.check_status(status)


def bench_float32() -> None:
    """The kernels of the true 32-bit path at SmolLM2-135M shapes: FMA products for a 2,048-token prompt and for 8
    decoded rows, split-key decode attention and one-warp-per-row attention over a float32 cache."""
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    for name, m, n, k in [("135m qkv, 2048 rows", 2048, 960, 576), ("135m gate/up, 2048 rows", 2048, 3072, 576),
                          ("135m down, 2048 rows", 2048, 576, 1536), ("135m qkv, 8 rows", 8, 960, 576),
                          ("135m head, 8 rows", 8, 49152, 576)]:
        a, w, c = torch.randn(m, k, device=DEV), torch.randn(n, k, device=DEV), torch.empty(m, n, device=DEV)
        t = graph_time(lambda: kernels.gemm_simt(a, w, c), reps=6)
        print(f"gemm_simt {name:24s} {m} x {n} x {k}: {t:8.1f} us {2.0 * m * n * k / t / 1e6:6.2f} TFLOP/s "
              f"{(m * k + n * k + m * n) * 4 / t / 1e3:6.0f} GB/s", flush=True)
    nh, nkv, hd, ps, ctx = 9, 3, 64, 16, 4096
    for m in (1, 8):
        per = ctx // ps
        kc = torch.randn(m * per + 4, nkv, ps, hd, device=DEV)
        vc = torch.randn_like(kc)
        tables = torch.arange(m * per, dtype=torch.int32, device=DEV).view(m, per).contiguous()
        row_seq = torch.arange(m, dtype=torch.int32, device=DEV)
        pos = torch.full((m,), ctx - 1, dtype=torch.int32, device=DEV)
        q = torch.randn(m, nh * hd, device=DEV)
        o = torch.empty_like(q)
        splits = kernels.decode_splits(m, nh, nkv, ctx)
        pa, pm = torch.empty(m * nh * splits * hd, device=DEV), torch.empty(m * nh * splits * 2, device=DEV)
        cn = torch.zeros(m * nh, dtype=torch.int32, device=DEV)
        nbytes = m * ctx * nkv * hd * 4 * 2
        t = graph_time(lambda: kernels.attention_decode(q, o, kc, vc, tables, row_seq, pos, nh, nkv, hd, ps, hd ** -0.5, None,
                                                        splits, pa, pm, cn, status))
        print(f"attention_decode (float32) batch {m} ctx {ctx} splits {splits}: {t:7.1f} us {nbytes / t / 1e3:6.0f} GB/s", flush=True)
        t = graph_time(lambda: kernels.attention_rows(q, o, kc, vc, tables, row_seq, pos, nh, nkv, hd, ps, hd ** -0.5, None, status))
        print(f"attention_rows   (float32) batch {m} ctx {ctx}: {t:7.1f} us {nbytes / t / 1e3:6.0f} GB/s", flush=True)
    kernels.check_status(status)


def bench_small() -> None:
    """The element-wise kernels and the sampling kernel at SmolLM2-135M sizes, for a 2,048-token prompt and for 8 rows."""
    from .parts.rope import rotary_table
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    d, inter, vocab, nh, nkv, hd, ps = 576, 1536, 49152, 9, 3, 64, 16
    table = (torch.randn(vocab, d, device=DEV) * 0.02).bfloat16()
    gain = torch.ones(d, device=DEV)
    rope = rotary_table(100000.0, hd, 8192).to(DEV)
    for n in (2048, 8):
        tokens = torch.randint(0, vocab, (n,), dtype=torch.int32, device=DEV)
        x = torch.empty(n, d, device=DEV)
        h = torch.empty(n, d, device=DEV, dtype=torch.bfloat16)
        t = graph_time(lambda: kernels.embed(table, tokens, x, status))
        print(f"embed            {n:5d} rows x {d}: {t:6.1f} us {n * d * 6 / t / 1e3:6.0f} GB/s", flush=True)
        t = graph_time(lambda: kernels.rmsnorm(x, gain, h, 1e-5))
        print(f"rmsnorm          {n:5d} rows x {d}: {t:6.1f} us {n * d * 6 / t / 1e3:6.0f} GB/s", flush=True)
        qkv = torch.randn(n, (nh + 2 * nkv) * hd, device=DEV).bfloat16()
        kc = torch.zeros(n // ps + 2, nkv, ps, hd, device=DEV, dtype=torch.bfloat16)
        vc = torch.zeros_like(kc)
        pos = torch.arange(n, dtype=torch.int32, device=DEV)
        t = graph_time(lambda: kernels.rope_kv_write(qkv, rope, pos, pos, kc, vc, nh, nkv, hd, hd, ps, True, status))
        print(f"rope_kv_write    {n:5d} rows: {t:6.1f} us {n * (nh + 2 * nkv) * hd * 2 * 2 / t / 1e3:6.0f} GB/s", flush=True)
        gu = torch.randn(n, 2 * inter, device=DEV).bfloat16()
        act = torch.empty(n, inter, device=DEV, dtype=torch.bfloat16)
        t = graph_time(lambda: kernels.swiglu(gu, act))
        print(f"swiglu           {n:5d} rows x {inter}: {t:6.1f} us {n * inter * 6 / t / 1e3:6.0f} GB/s", flush=True)
    for rows in (1, 8, 64):
        logits = torch.randn(rows, vocab, device=DEV)
        out = torch.empty(rows, dtype=torch.int32, device=DEV)
        temp = torch.full((rows,), 0.8, device=DEV)
        unif = torch.rand(rows, device=DEV)
        t = graph_time(lambda: kernels.sample(logits, out))
        t2 = graph_time(lambda: kernels.sample(logits, out, temp, unif))
        print(f"sample           {rows:3d} rows x {vocab}: greedy {t:6.1f} us {rows * vocab * 4 / t / 1e3:6.0f} GB/s | temperature "
              f"{t2:6.1f} us {rows * vocab * 4 * 3 / t2 / 1e3:6.0f} GB/s (three passes)", flush=True)
    kernels.check_status(status)


def bench_decode_program(batches) -> None:
    """A decode step of SmolLM2-135M shapes at context 4096: as the chain of kernels in a CUDA graph, and as a decode
    program run by the persistent kernel, shared by operations and by rows; for the programs also where the time goes
    (clock values that the first block notes for each operation: its own share of the work including the wait for the
    operation before, and the arrival at the barrier behind it), averaged over the layers."""
    import shutil
    import tempfile

    import numpy as np

    from . import write_random_model
    from .engine.engine import Engine, StepEntry
    from .models.llama import make_llama_raw_config
    shape = dict(num_hidden_layers=30, hidden_size=576, num_attention_heads=9, num_key_value_heads=3, intermediate_size=1536,
                 vocab_size=49152, rope_theta=100000.0, rms_norm_eps=1e-5, tie_word_embeddings=True, max_position_embeddings=8192)
    ctx_len, steps = 4096, 48
    tmp = tempfile.mkdtemp(prefix="glassbox_b200_microbench_")
    try:
        write_random_model(tmp, make_llama_raw_config(**shape), 0, torch.bfloat16)
        rng = np.random.default_rng(0)
        for batch in batches or (1, 8):
            for label, how in (("kernel chain", None), ("program, by operations", kernels.BY_OPERATIONS),
                               ("program, by rows", kernels.BY_ROWS)):
                kernels.PROGRAM_HOW = how if how is not None else kernels.BY_ROWS
                eng = Engine(tmp, "bfloat16", cache_tokens=batch * (ctx_len + 64), max_batch_tokens=2048, max_requests=batch + 2,
                             use_programs=how is not None)
                for i in range(batch):
                    eng.add_request(i)
                    toks = rng.integers(0, shape["vocab_size"], size=ctx_len - steps - 8)
                    for j in range(0, len(toks), 2048):
                        eng.step([StepEntry(i, toks[j:j + 2048].tolist(), [])])
                flags = [1] * batch

                def one():
                    eng.step([StepEntry(i, [5], [0]) for i in range(batch)], sampling=flags)
                for _ in range(4):
                    one()
                torch.cuda.synchronize()
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                for _ in range(steps):
                    one()
                e1.record()
                torch.cuda.synchronize()
                line = f"135m batch {batch} context {ctx_len} {label:24s}: {e0.elapsed_time(e1) / steps:7.4f} ms per step"
                if how is not None:     # one more step outside the graphs, traced
                    eng.use_graphs = False
                    eng.ctx.program.trace_next = True
                    one()
                    torch.cuda.synchronize()
                    n, trace, _ = max(eng.ctx.program.traces, key=lambda t: t[0])
                    t = trace.cpu().numpy().reshape(2, n, 4).astype(np.float64)[0] / 1965.0     # microseconds at 1,965 MHz
                    k = (n // 5) * 5
                    parts = []
                    for j, name in enumerate(("qkv", "attention", "o", "gate/up", "down")):
                        sel = t[j:k:5]
                        parts.append(f"{name} {np.mean(sel[:, 2] - sel[:, 0]):.1f}+{np.mean((sel[:, 3] - sel[:, 2])[:-1]):.1f}")
                    line += f" | per operation, us (work + arrival), {n} operations: " + ", ".join(parts)
                print(line, flush=True)
                del eng
    finally:
        shutil.rmtree(tmp, ignore_errors=True)


def bench_layer_gemms(rows) -> None:
    """The four products of one SmolLM2-135M decode layer with what the layer folds into them: the norm on the way in,
    rotation and cache write on the way out of QKV, SwiGLU, the residual additions; each alone (back to back in a
    graph, cold weights) and the four in a row."""
    from .parts.rope import rotary_table
    st = torch.zeros(1, dtype=torch.int32, device=DEV)
    d, inter, nh, nkv, hd, ps = 576, 1536, 9, 3, 64, 16
    for m in rows or (1, 8, 16):
        res = torch.randn(m, d, device=DEV)
        gain = torch.ones(d, device=DEV)
        xb = torch.randn(m, d, device=DEV).bfloat16()
        wq, wo, wg, wd = _rotating(960, d), _rotating(d, d), _rotating(2 * inter, d), _rotating(d, inter)
        qkv = torch.empty(m, 960, device=DEV, dtype=torch.bfloat16)
        act = torch.empty(m, inter, device=DEV, dtype=torch.bfloat16)
        table = rotary_table(1e5, hd, 8192).to(DEV)
        pos = torch.full((m,), 4000, dtype=torch.int32, device=DEV)
        slots = torch.arange(m, dtype=torch.int32, device=DEV) * ps
        kc = torch.zeros(m + 2, nkv, ps, hd, device=DEV, dtype=torch.bfloat16)
        vc = torch.zeros_like(kc)
        turn = [0]

        def nxt(ws):
            turn[0] += 1
            return ws[turn[0] % len(ws)]

        def qkv_full():
            kernels.gemm_stream_qkv(res, nxt(wq), qkv, table, pos, slots, kc, vc, nh, nkv, hd, ps, True, st, norm=(gain, 1e-5))

        def layer():
            qkv_full()
            kernels.gemm_stream(qkv[:, :d], nxt(wo), res, True)
            kernels.gemm_stream(res, nxt(wg), act, gated=True, norm=(gain, 1e-5))
            kernels.gemm_stream(act, nxt(wd), res, True)

        t = [graph_time(lambda: kernels.gemm_stream(xb, nxt(wq), qkv)),
             graph_time(lambda: kernels.gemm_stream(res, nxt(wq), qkv, norm=(gain, 1e-5))),
             graph_time(qkv_full),
             graph_time(lambda: kernels.gemm_stream(xb, nxt(wo), res, True)),
             graph_time(lambda: kernels.gemm_stream(xb, nxt(wg), act, gated=True)),
             graph_time(lambda: kernels.gemm_stream(res, nxt(wg), act, gated=True, norm=(gain, 1e-5))),
             graph_time(lambda: kernels.gemm_stream(act, nxt(wd), res, True)),
             graph_time(layer, reps=8)]
        print(f"rows {m:2d}: qkv {t[0]:.2f} us, + norm {t[1]:.2f}, + rotation and cache write {t[2]:.2f} | o + residual {t[3]:.2f} | "
              f"gate/up + SwiGLU {t[4]:.2f}, + norm {t[5]:.2f} | down + residual {t[6]:.2f} | the four in a row {t[7]:.2f}", flush=True)
    kernels.check_status(st)


CASES = ("gemm_stream", "gemm_tc", "attention_decode", "attention_splits", "attention_prefill", "float32", "small", "decode_program", "layer_gemms")


def main(argv) -> int:
    global ONCE
    if "--once" in argv:
        ONCE = True
        argv = [a for a in argv if a != "--once"]
    if not argv or argv[0] not in CASES or (argv[0] == "attention_splits" and len(argv) < 4):
        print(__doc__)
        return 2
    torch.cuda.set_device(0)
    kernels.lib()
    if argv[0] == "gemm_stream":
        bench_gemm_stream(argv[1:])
    elif argv[0] == "gemm_tc":
        bench_gemm_tc()
    elif argv[0] == "attention_decode":
        bench_attention_decode([int(x) for x in argv[1:]])
    elif argv[0] == "attention_splits":
        nh, nkv, m = (int(x) for x in argv[1:4])
        bench_attention_decode([m], nh, nkv, int(argv[4]) if len(argv) > 4 else 4096, sweep=True)
    elif argv[0] == "float32":
        bench_float32()
    elif argv[0] == "small":
        bench_small()
    elif argv[0] == "decode_program":
        bench_decode_program([int(x) for x in argv[1:]])
    elif argv[0] == "layer_gemms":
        bench_layer_gemms([int(x) for x in argv[1:]])
    else:
        bench_attention_prefill()
    return 0


if __name__ == "__main__":
    sys.exit(main(sys.argv[1:]))
