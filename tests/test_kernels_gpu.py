"""Each CUDA kernel alone against a plain float32/float64 PyTorch statement of the same operation, at
sizes other than the engine's: awkward lengths, head sizes in steps of 16, any number of heads and
groups, widths and vocabularies that are no power of two (after the method of
crates/glassbox-core/src/kernels.rs:675-720)."""
import math
import random

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

DEV = "cuda:0"
DTYPES = [torch.float32, torch.bfloat16]


def tol(dtype, scale=1.0):
    return (2e-5 if dtype == torch.float32 else 1.6e-2) * scale


def status():
    return torch.zeros(1, dtype=torch.int32, device=DEV)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("n, d, vocab", [(1, 16, 7), (5, 576, 301), (33, 100, 49153)])
def test_embed(dtype, n, d, vocab):
    from glassbox_b200 import kernels
    table = torch.randn(vocab, d, device=DEV).to(dtype)
    toks = torch.randint(0, vocab, (n,), device=DEV, dtype=torch.int32)
    x = torch.empty(n, d, device=DEV)
    st = status()
    kernels.embed(table, toks, x, st)
    assert torch.equal(x, table[toks.long()].float()) and int(st) == 0
    toks[0] = vocab
    kernels.embed(table, toks, x, st)
    assert int(st) == 1 and float(x[0].abs().max()) == 0.0


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("n, d, eps", [(1, 7, 1e-5), (3, 576, 1e-6), (17, 1537, 3e-6), (9, 8192, 1e-5),
                                       (2048, 576, 1e-5), (13, 2048, 1e-5), (5, 4096, 1e-6), (21, 132, 1e-5)])
def test_rmsnorm(dtype, n, d, eps):
    from glassbox_b200 import kernels
    x = torch.randn(n + 3, d, device=DEV) * 3
    gain = 1 + 0.1 * torch.randn(d, device=DEV)
    rows = torch.randperm(n + 3, device=DEV)[:n].to(torch.int32)
    out = torch.empty(n, d, device=DEV, dtype=dtype)
    kernels.rmsnorm(x, gain, out, eps, rows)
    xs = x[rows.long()].double()
    ref = gain.double() * (xs / torch.sqrt((xs * xs).mean(-1, keepdim=True) + eps))
    assert (out.double() - ref).abs().max() <= tol(dtype, 4)
    out2 = torch.empty(n + 3, d, device=DEV, dtype=dtype)
    kernels.rmsnorm(x, gain, out2, eps)
    assert torch.equal(out2[rows.long()], out)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("n, inter", [(1, 1), (3, 176), (17, 1537)])
def test_swiglu(dtype, n, inter):
    from glassbox_b200 import kernels
    gu = (torch.randn(n, 2 * inter, device=DEV) * 2).to(dtype)
    act = torch.empty(n, inter, device=DEV, dtype=dtype)
    kernels.swiglu(gu, act)
    g, u = gu[:, :inter].double(), gu[:, inter:].double()
    ref = g / (1 + torch.exp(-g)) * u
    assert ((act.double() - ref).abs() / (1 + ref.abs())).max() <= tol(dtype, 1)      # relative: values reach ~50


@pytest.mark.parametrize("a_dt, w_dt, c_dt", [(torch.float32,) * 3, (torch.bfloat16,) * 3,
                                              (torch.bfloat16, torch.bfloat16, torch.float32),
                                              (torch.bfloat16, torch.float32, torch.bfloat16)])
@pytest.mark.parametrize("M, N, K", [(1, 32, 32), (1, 7, 1537), (2, 100, 33), (3, 960, 576), (8, 17, 31),
                                     (9, 65, 63), (17, 160, 50), (70, 130, 100), (128, 49, 576)])
def test_gemm_simt(a_dt, w_dt, c_dt, M, N, K):
    from glassbox_b200 import kernels
    a = torch.randn(M, K, device=DEV).to(a_dt)
    w = (torch.randn(N, K, device=DEV) / math.sqrt(K)).to(w_dt)
    c = torch.empty(M, N, device=DEV, dtype=c_dt)
    kernels.gemm_simt(a, w, c)
    ref = a.double() @ w.double().T
    assert (c.double() - ref).abs().max() <= tol(c_dt, 2)
    if c_dt == torch.float32:
        base = torch.randn(M, N, device=DEV)
        c2 = base.clone()
        kernels.gemm_simt(a, w, c2, accumulate=True)
        assert (c2.double() - (base.double() + ref)).abs().max() <= tol(c_dt, 2)
    # strided operands: a and c are column slices of wider buffers (as q inside qkv)
    wide_a = torch.randn(M, K + 8, device=DEV).to(a_dt)
    wide_c = torch.zeros(M, N + 5, device=DEV, dtype=c_dt)
    kernels.gemm_simt(wide_a[:, 8:], w, wide_c[:, :N])
    assert (wide_c[:, :N].double() - wide_a[:, 8:].double() @ w.double().T).abs().max() <= tol(c_dt, 2)
    assert float(wide_c[:, N:].abs().max()) == 0.0


def test_gemm_simt_rows_do_not_depend_on_the_batch():
    """The float32 product of a row is bit-identical whatever else is in the batch (same kernel)."""
    from glassbox_b200 import kernels
    a = torch.randn(8, 576, device=DEV)
    w = torch.randn(200, 576, device=DEV)
    full = torch.empty(8, 200, device=DEV)
    kernels.gemm_simt(a, w, full)
    for m in (1, 3):
        part = torch.empty(m, 200, device=DEV)
        kernels.gemm_simt(a[:m].contiguous(), w, part)
        assert torch.equal(part, full[:m])


def make_cache(dtype, n_seqs, lens, nkv, hd, page_size, extra_pages=3, seed=0):
    """Random K/V scattered over shuffled pages; returns cache tensors, tables, and dense copies."""
    g = torch.Generator(device="cpu").manual_seed(seed)
    pages_per = [-(-l // page_size) for l in lens]
    num_pages = sum(pages_per) + extra_pages
    perm = torch.randperm(num_pages, generator=g).tolist()
    k = torch.randn(num_pages, nkv, page_size, hd, generator=g).to(dtype)
    v = torch.randn(num_pages, nkv, page_size, hd, generator=g).to(dtype)
    max_pages = max(pages_per) + 1
    tables = torch.full((n_seqs, max_pages), -1, dtype=torch.int32)
    dense = []
    at = 0
    for s, l in enumerate(lens):
        ids = perm[at:at + pages_per[s]]
        at += pages_per[s]
        tables[s, :len(ids)] = torch.tensor(ids, dtype=torch.int32)
        kk = torch.cat([k[p] for p in ids], dim=1)[:, :l].double()      # [nkv, l, hd]
        vv = torch.cat([v[p] for p in ids], dim=1)[:, :l].double()
        dense.append((kk, vv))
    return k.to(DEV), v.to(DEV), tables.to(DEV), dense


def ref_attention(q, dense, row_seq, positions, nh, nkv, scale, window):
    out = torch.zeros(q.shape[0], nh, q.shape[-1], dtype=torch.float64)
    group = nh // nkv
    for r in range(q.shape[0]):
        kk, vv = dense[row_seq[r]]
        p = positions[r]
        lo = max(0, p + 1 - window) if window else 0
        for h in range(nh):
            s = (kk[h // group, lo:p + 1] @ q[r, h].double()) * scale
            out[r, h] = torch.softmax(s, dim=0) @ vv[h // group, lo:p + 1]
    return out


ATT_CASES = [  # nh, nkv, hd, page_size, window, lens
    (4, 2, 16, 16, None, [5, 17, 33]),
    (3, 1, 32, 16, None, [1, 100, 64, 257]),
    (5, 5, 48, 16, 37, [300, 48, 17]),
    (9, 3, 64, 32, None, [700, 65]),
    (12, 2, 80, 16, 100, [130, 250]),       # six query heads per kv head: two sub-groups
    (2, 1, 256, 64, None, [129]),
]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("case", ATT_CASES)
def test_attention_rows(dtype, case):
    from glassbox_b200 import kernels
    nh, nkv, hd, ps, window, lens = case
    k, v, tables, dense = make_cache(dtype, len(lens), lens, nkv, hd, ps)
    rng = random.Random(1)
    row_seq, positions = [], []
    for s, l in enumerate(lens):                       # several rows per sequence, anywhere in it
        for p in sorted({0, l - 1, l // 2, rng.randrange(l), min(l - 1, ps - 1), min(l - 1, ps)}):
            row_seq.append(s)
            positions.append(p)
    n = len(row_seq)
    q = torch.randn(n, nh, hd).to(dtype)
    qd = q.to(DEV).reshape(n, nh * hd)
    out = torch.empty(n, nh * hd, device=DEV, dtype=dtype)
    st = status()
    kernels.attention_rows(qd, out, k, v, tables, torch.tensor(row_seq, dtype=torch.int32, device=DEV),
                           torch.tensor(positions, dtype=torch.int32, device=DEV), nh, nkv, hd, ps, hd ** -0.5, window, st)
    ref = ref_attention(q, dense, row_seq, positions, nh, nkv, hd ** -0.5, window)
    assert int(st) == 0
    assert (out.cpu().double().reshape(n, nh, hd) - ref).abs().max() <= tol(dtype, 2)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("splits", [1, 2, 5, 40])
@pytest.mark.parametrize("case", ATT_CASES)
def test_attention_decode(dtype, case, splits):
    from glassbox_b200 import kernels
    nh, nkv, hd, ps, window, lens = case
    k, v, tables, dense = make_cache(dtype, len(lens), lens, nkv, hd, ps, seed=2)
    n = len(lens) + 1                                      # one row per sequence, plus a padding row
    row_seq = list(range(len(lens))) + [0]
    positions = [l - 1 for l in lens] + [-1]
    q = torch.randn(n, nh, hd).to(dtype)
    out = torch.full((n, nh * hd), 7.0, device=DEV, dtype=dtype)
    part_acc = torch.empty(n * nh * splits * hd, device=DEV)
    part_ml = torch.empty(n * nh * splits * 2, device=DEV)
    counters = torch.zeros(n * nh, dtype=torch.int32, device=DEV)
    st = status()
    for _ in range(2):                                     # twice: the counters must come back to zero
        kernels.attention_decode(q.to(DEV).reshape(n, nh * hd), out, k, v, tables,
                                 torch.tensor(row_seq, dtype=torch.int32, device=DEV),
                                 torch.tensor(positions, dtype=torch.int32, device=DEV), nh, nkv, hd, ps, hd ** -0.5,
                                 window, splits, part_acc, part_ml, counters, st)
        ref = ref_attention(q[:-1], dense, row_seq[:-1], positions[:-1], nh, nkv, hd ** -0.5, window)
        got = out.cpu().double().reshape(n, nh, hd)
        assert int(st) == 0 and int(counters.abs().max()) == 0
        assert (got[:-1] - ref).abs().max() <= tol(dtype, 2)
        assert float(got[-1].abs().max()) == 0.0            # the padding row is zeroed, nothing else
        out.fill_(7.0)


@pytest.mark.parametrize("dtype", DTYPES)
def test_attention_one_far_key_stands_out(dtype):
    """Among hundreds of keys one far key's score stands out by 30: the output must be its value,
    through either kernel, wherever the page boundary falls."""
    from glassbox_b200 import kernels
    nh, nkv, hd, ps = 2, 1, 64, 16
    for far in (0, 15, 16, 250, 499):
        L = 500
        k, v, tables, dense = make_cache(dtype, 1, [L], nkv, hd, ps, seed=far)
        q = torch.zeros(1, nh, hd)
        kk, vv = dense[0]
        q[0, :] = (kk[0, far] / kk[0, far].norm() ** 2 * 60.0 * 8.0).float()   # score 60 at `far`, ~N(0, 8) elsewhere
        q = q.to(dtype)
        ref = ref_attention(q, dense, [0], [L - 1], nh, nkv, hd ** -0.5, None)
        assert (ref[0, 0] - vv[0, far]).abs().max() < 1e-3, "the crafted score does not dominate"
        args = (k, v, tables, torch.zeros(1, dtype=torch.int32, device=DEV),
                torch.tensor([L - 1], dtype=torch.int32, device=DEV), nh, nkv, hd, ps, hd ** -0.5, None)
        out = torch.empty(1, nh * hd, device=DEV, dtype=dtype)
        kernels.attention_rows(q.to(DEV).reshape(1, -1), out, *args, status())
        assert (out.cpu().double().reshape(nh, hd) - ref[0]).abs().max() <= tol(dtype, 2)
        splits = 4
        kernels.attention_decode(q.to(DEV).reshape(1, -1), out, *args, splits, torch.empty(nh * splits * hd, device=DEV),
                                 torch.empty(nh * splits * 2, device=DEV), torch.zeros(nh, dtype=torch.int32, device=DEV),
                                 status())
        assert (out.cpu().double().reshape(nh, hd) - ref[0]).abs().max() <= tol(dtype, 2)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("nh, nkv, hd, rot, ps", [(4, 2, 16, 16, 16), (3, 1, 32, 32, 16), (5, 5, 48, 24, 32), (9, 3, 64, 64, 16)])
def test_rope_and_cache_write(dtype, nh, nkv, hd, rot, ps):
    from glassbox_b200 import kernels
    from glassbox_b200.parts.rope import rotary_table
    from plain.llama_plain import rope_angles
    n, max_pos, pages = 11, 300, 9
    table = rotary_table(123456.0, rot, max_pos).to(DEV)
    qkv = torch.randn(n, (nh + 2 * nkv) * hd).to(dtype)
    positions = torch.tensor([0, 1, 2, 17, 299, 150, 31, 32, 33, -1, 64], dtype=torch.int32)
    slots = torch.tensor([5, 0, 143, 17, 100, 33, 64, 65, 66, -1, 1], dtype=torch.int32)
    kc = torch.zeros(pages, nkv, ps, hd, device=DEV, dtype=dtype)
    vc = torch.zeros_like(kc)
    dev = qkv.to(DEV).clone()
    st = status()
    kernels.rope_kv_write(dev, table, positions.to(DEV), slots.to(DEV), kc, vc, nh, nkv, hd, rot, ps, True, st)
    assert int(st) == 0
    got = dev.cpu().double()
    cos, sin = rope_angles(positions.clamp(min=0).numpy(), rot, float(np.float32(123456.0)))
    src = qkv.double()
    for r in range(n):
        if positions[r] < 0:                                # padding row: untouched, nothing stored
            assert torch.equal(got[r], src[r])
            continue
        heads = src[r, :(nh + nkv) * hd].reshape(nh + nkv, hd).clone()
        x0, x1 = heads[:, :rot // 2].clone(), heads[:, rot // 2:rot].clone()
        c, s = torch.from_numpy(cos[r]), torch.from_numpy(sin[r])
        heads[:, :rot // 2] = x0 * c - x1 * s
        heads[:, rot // 2:rot] = x1 * c + x0 * s
        assert (got[r, :(nh + nkv) * hd].reshape(nh + nkv, hd) - heads).abs().max() <= tol(dtype, 4)
        page, off = int(slots[r]) // ps, int(slots[r]) % ps
        assert (kc[page, :, off].cpu().double() - heads[nh:]).abs().max() <= tol(dtype, 4)
        assert torch.equal(vc[page, :, off].cpu(), qkv[r, (nh + nkv) * hd:].reshape(nkv, hd))
    written = {int(s) for s, p in zip(slots, positions) if p >= 0}
    mask = torch.ones(pages * ps, dtype=torch.bool)
    mask[list(written)] = False
    assert float(kc.permute(0, 2, 1, 3).reshape(pages * ps, -1)[mask.to(DEV)].abs().max()) == 0.0
    # bad indices are recorded and skipped, never followed
    bad = status()
    kernels.rope_kv_write(dev, table, torch.full((n,), 300, dtype=torch.int32, device=DEV), slots.to(DEV).abs(), kc, vc,
                          nh, nkv, hd, rot, ps, True, bad)
    assert int(bad) & 4
    bad.zero_()
    kernels.rope_kv_write(dev, table, positions.to(DEV).clamp(min=0), torch.full((n,), pages * ps, dtype=torch.int32, device=DEV),
                          kc, vc, nh, nkv, hd, rot, ps, True, bad)
    assert int(bad) & 2


@pytest.mark.parametrize("vocab", [5, 256, 49152, 50001])
def test_sampling(vocab):
    from glassbox_b200 import kernels
    from plain import sampler_plain
    rows = 6
    g = torch.Generator().manual_seed(vocab)
    logits = torch.randn(rows, vocab, generator=g) * 3
    logits[1, vocab // 2] = logits[1].max() + 1
    logits[2, 3] = logits[2, vocab - 1] = logits[2].max() + 2          # a tie: the first index wins
    out = torch.empty(rows, dtype=torch.int32, device=DEV)
    kernels.sample(logits.to(DEV), out)
    assert out.tolist() == [int(torch.argmax(r)) for r in logits] and out[2] == 3
    temps = torch.tensor([0.0, 0.8, 1.0, 1.7, 0.3, 1.0])
    for trial in range(20):
        unif = torch.rand(rows, generator=g)
        kernels.sample(logits.to(DEV), out, temps.to(DEV), unif.to(DEV))
        for r in range(rows):
            dist = sampler_plain.distribution(logits[r].tolist(), [], temperature=float(temps[r]))
            want = sampler_plain.draw(dist, float(unif[r]))
            if int(out[r]) != want:                     # only an edge of the cumulative sum may differ
                acc = 0.0
                for t in sorted(dist):
                    acc += dist[t]
                    if t in (int(out[r]), want):
                        assert abs(acc - float(unif[r])) < 1e-4 or abs(acc - dist[t] - float(unif[r])) < 1e-4
                        break


def test_copy_pages():
    from glassbox_b200 import kernels
    k = torch.randn(3, 10, 2, 16, 48, device=DEV).to(torch.bfloat16)
    v = torch.randn_like(k)
    k0, v0 = k.clone(), v.clone()
    kernels.copy_pages(k, v, torch.tensor([[1, 7], [4, 0]], dtype=torch.int32, device=DEV))
    for src, dst in ((1, 7), (4, 0)):
        assert torch.equal(k[:, dst], k0[:, src]) and torch.equal(v[:, dst], v0[:, src])
    keep = [p for p in range(10) if p not in (7, 0)]
    assert torch.equal(k[:, keep], k0[:, keep])


def test_sizes_outside_the_kernels_range_are_refused():
    from glassbox_b200 import kernels
    q = torch.zeros(1, 2 * 24, device=DEV)
    kc = torch.zeros(4, 1, 16, 24, device=DEV)
    with pytest.raises(kernels.KernelError, match="multiple of 16"):
        kernels.attention_decode(q, q.clone(), kc, kc, torch.zeros(1, 4, dtype=torch.int32, device=DEV),
                                 torch.zeros(1, dtype=torch.int32, device=DEV), torch.zeros(1, dtype=torch.int32, device=DEV),
                                 2, 1, 24, 16, 1.0, None, 1, None, None, None, status())
    with pytest.raises(kernels.KernelError, match="multiple"):
        kernels.attention_rows(torch.zeros(1, 3 * 16, device=DEV), torch.zeros(1, 3 * 16, device=DEV),
                               torch.zeros(4, 2, 16, 16, device=DEV), torch.zeros(4, 2, 16, 16, device=DEV),
                               torch.zeros(1, 4, dtype=torch.int32, device=DEV), torch.zeros(1, dtype=torch.int32, device=DEV),
                               torch.zeros(1, dtype=torch.int32, device=DEV), 3, 2, 16, 16, 1.0, None, status())
    with pytest.raises(kernels.KernelError):
        kernels.gemm_simt(torch.zeros(2, 4), torch.zeros(3, 4), torch.zeros(2, 3))      # CPU tensors: no CPU path


@pytest.mark.parametrize("M", [1, 2, 7, 8, 9, 16, 31, 33, 64])
@pytest.mark.parametrize("N, K", [(16, 8), (100, 40), (576, 576), (960, 264), (49, 1544), (3072, 576),
                                  (576, 1536), (960, 2560), (2048, 2048), (40, 8200)])   # the last four: K split over a cluster
def test_gemm_stream(M, N, K):
    from glassbox_b200 import kernels
    a = torch.randn(M, K, device=DEV).to(torch.bfloat16)
    w = (torch.randn(N, K, device=DEV) / math.sqrt(K)).to(torch.bfloat16)
    assert kernels.gemm_stream_supported(a, w)
    ref = a.double() @ w.double().T
    c = torch.empty(M, N, device=DEV, dtype=torch.bfloat16)
    kernels.gemm_stream(a, w, c)
    assert (c.double() - ref).abs().max() <= tol(torch.bfloat16, 2)
    c32 = torch.empty(M, N, device=DEV)
    kernels.gemm_stream(a, w, c32)
    assert (c32.double() - ref).abs().max() <= 2e-5 * math.sqrt(K)
    base = torch.randn(M, N, device=DEV)
    acc = base.clone()
    kernels.gemm_stream(a, w, acc, accumulate=True)
    assert (acc.double() - base.double() - ref).abs().max() <= 2e-5 * math.sqrt(K)
    # the same row gives the same bits whatever else is in the batch and wherever it stands in it
    other = torch.randn(M, K, device=DEV).to(torch.bfloat16)
    place = M // 2
    other[place] = a[0]
    moved = torch.empty(M, N, device=DEV)
    kernels.gemm_stream(other, w, moved)
    assert torch.equal(moved[place], c32[0])


@pytest.mark.parametrize("M", [1, 5, 8, 24, 64])
@pytest.mark.parametrize("inter, K", [(16, 16), (176, 64), (1536, 576), (48, 1000), (256, 2048), (48, 4104)])
def test_gemm_stream_gated(M, inter, K):
    from glassbox_b200 import kernels
    a = torch.randn(M, K, device=DEV).to(torch.bfloat16)
    w = (torch.randn(2 * inter, K, device=DEV) * (2.0 / math.sqrt(K))).to(torch.bfloat16)
    act = torch.empty(M, inter, device=DEV, dtype=torch.bfloat16)
    kernels.gemm_stream(a, w, act, gated=True)
    gu = a.double() @ w.double().T
    g, u = gu[:, :inter], gu[:, inter:]
    ref = g / (1 + torch.exp(-g)) * u
    assert ((act.double() - ref).abs() / (1 + ref.abs())).max() <= tol(torch.bfloat16, 1)   # relative: values reach ~10


def test_gemm_stream_refuses_what_it_cannot_do():
    from glassbox_b200 import kernels
    a = torch.zeros(65, 64, device=DEV, dtype=torch.bfloat16)
    w = torch.zeros(32, 64, device=DEV, dtype=torch.bfloat16)
    assert not kernels.gemm_stream_supported(a, w)
    assert not kernels.gemm_stream_supported(a[:4, :60], w[:, :60])
    with pytest.raises(kernels.KernelError, match="M <= 64"):
        kernels.gemm_stream(a, w, torch.zeros(65, 32, device=DEV))


MMA_CASES = [  # nh, nkv, hd, page_size, window, lens
    (4, 2, 16, 16, None, [5, 17, 33, 64]),
    (3, 1, 32, 16, None, [1, 100, 64, 257]),
    (9, 3, 64, 16, None, [700, 65, 31, 32, 33]),
    (9, 3, 64, 32, 100, [700, 99, 100, 101]),
    (32, 2, 64, 16, None, [300]),                # sixteen query heads per kv head
    (5, 5, 128, 64, 37, [300, 48, 17]),
    (2, 1, 128, 16, None, [129, 1000]),
]


@pytest.mark.parametrize("warps", [4, 8])
@pytest.mark.parametrize("splits", [1, 3, 16])
@pytest.mark.parametrize("case", MMA_CASES)
def test_attention_decode_mma(case, splits, warps):
    from glassbox_b200 import kernels
    nh, nkv, hd, ps, window, lens = case
    dtype = torch.bfloat16
    assert kernels.attention_decode_mma_supported(dtype, nh, nkv, hd)
    if warps == 8 and hd != 64:
        pytest.skip("eight warps per block are built for head size 64")
    k, v, tables, dense = make_cache(dtype, len(lens), lens, nkv, hd, ps, seed=3)
    n = len(lens) + 1
    row_seq = list(range(len(lens))) + [0]
    positions = [l - 1 for l in lens] + [-1]
    q = torch.randn(n, nh, hd).to(dtype)
    out = torch.full((n, nh * hd), 7.0, device=DEV, dtype=dtype)
    part_acc = torch.empty(n * nh * warps * splits * hd, device=DEV)
    part_ml = torch.empty(n * nh * warps * splits * 2, device=DEV)
    counters = torch.zeros(n * nkv, dtype=torch.int32, device=DEV)
    st = status()
    ref = ref_attention(q[:-1], dense, row_seq[:-1], positions[:-1], nh, nkv, hd ** -0.5, window)
    for _ in range(2):
        kernels.attention_decode_mma(q.to(DEV).reshape(n, nh * hd), out, k, v, tables,
                                     torch.tensor(row_seq, dtype=torch.int32, device=DEV),
                                     torch.tensor(positions, dtype=torch.int32, device=DEV), nh, nkv, hd, ps, hd ** -0.5,
                                     window, splits, part_acc, part_ml, counters, st, 0, warps)
        got = out.cpu().double().reshape(n, nh, hd)
        assert int(st) == 0 and int(counters.abs().max()) == 0
        assert (got[:-1] - ref).abs().max() <= tol(dtype, 2)
        assert float(got[-1].abs().max()) == 0.0
        out.fill_(7.0)


def test_attention_decode_mma_one_far_key_stands_out():
    from glassbox_b200 import kernels
    nh, nkv, hd, ps, dtype = 6, 2, 64, 16, torch.bfloat16
    for far in (0, 15, 16, 31, 32, 250, 499):
        L = 500
        k, v, tables, dense = make_cache(dtype, 1, [L], nkv, hd, ps, seed=far)
        kk, vv = dense[0]
        q = torch.zeros(1, nh, hd)
        for h in range(nh):                         # heads of kv head 0 look for `far`, of kv head 1 for far/2
            target = far if h < 3 else far // 2
            key = kk[h // 3, target]
            q[0, h] = (key / key.norm() ** 2 * 60.0 * 8.0).float()
        q = q.to(dtype)
        ref = ref_attention(q, dense, [0], [L - 1], nh, nkv, hd ** -0.5, None)
        assert (ref[0, 0] - vv[0, far]).abs().max() < 1e-3 and (ref[0, 5] - vv[1, far // 2]).abs().max() < 1e-3
        out = torch.empty(1, nh * hd, device=DEV, dtype=dtype)
        splits = 3
        kernels.attention_decode_mma(q.to(DEV).reshape(1, -1), out, k, v, tables, torch.zeros(1, dtype=torch.int32, device=DEV),
                                     torch.tensor([L - 1], dtype=torch.int32, device=DEV), nh, nkv, hd, ps, hd ** -0.5, None,
                                     splits, torch.empty(nh * 4 * splits * hd, device=DEV),
                                     torch.empty(nh * 4 * splits * 2, device=DEV),
                                     torch.zeros(nkv, dtype=torch.int32, device=DEV), status())
        assert (out.cpu().double().reshape(nh, hd) - ref[0]).abs().max() <= tol(dtype, 2)


@pytest.mark.parametrize("M, N, K", [(128, 128, 64), (128, 64, 128), (65, 960, 576), (200, 576, 576), (2048, 3072, 576),
                                     (300, 100, 72), (129, 49160, 576), (1000, 576, 1536), (77, 8, 8), (256, 200, 1000),
                                     (33, 4096, 1024), (17, 16384, 64), (1, 128, 64)])   # few rows: a partly empty tile
def test_gemm_tcgen05(M, N, K):
    from glassbox_b200 import kernels
    a = torch.randn(M, K, device=DEV).to(torch.bfloat16)
    w = (torch.randn(N, K, device=DEV) / math.sqrt(K)).to(torch.bfloat16)
    st = status()
    assert kernels.gemm_tc_supported(a, w, torch.empty(M, N, device=DEV))
    ref = a.double() @ w.double().T
    c32 = torch.full((M, N), 9.0, device=DEV)
    kernels.gemm_tc(a, w, c32, status=st)
    assert int(st) == 0, "a bounded wait inside the kernel gave up"
    assert (c32.double() - ref).abs().max() <= 2e-5 * math.sqrt(K) + 1e-6
    c16 = torch.empty(M, N, device=DEV, dtype=torch.bfloat16)
    kernels.gemm_tc(a, w, c16, status=st)
    assert (c16.double() - ref).abs().max() <= tol(torch.bfloat16, 2)
    base = torch.randn(M, N, device=DEV)
    acc = base.clone()
    kernels.gemm_tc(a, w, acc, accumulate=True, status=st)
    assert (acc.double() - base.double() - ref).abs().max() <= 2e-5 * math.sqrt(K) + 1e-6
    # strided views: a is a column slice of a wider buffer, c a slice of a wider output
    wide_a = torch.randn(M, K + 16, device=DEV).to(torch.bfloat16)
    wide_c = torch.zeros(M, N + 3, device=DEV)
    kernels.gemm_tc(wide_a[:, 16:], w, wide_c[:, :N], status=st)
    assert (wide_c[:, :N].double() - wide_a[:, 16:].double() @ w.double().T).abs().max() <= 2e-5 * math.sqrt(K) + 1e-6
    assert float(wide_c[:, N:].abs().max()) == 0.0 and int(st) == 0


def test_gemm_tcgen05_refuses_misaligned_operands():
    from glassbox_b200 import kernels
    a = torch.zeros(128, 68, device=DEV, dtype=torch.bfloat16)
    w = torch.zeros(64, 68, device=DEV, dtype=torch.bfloat16)
    assert not kernels.gemm_tc_supported(a, w, torch.empty(128, 64, device=DEV))          # row stride 68 is no multiple of 8
    assert not kernels.gemm_tc_supported(a[:, 1:65], w[:, 1:65], torch.empty(128, 64, device=DEV))
    with pytest.raises(kernels.KernelError, match="aligned"):
        kernels.gemm_tc(a, w, torch.empty(128, 64, device=DEV))


PREFILL_CASES = [  # nh, nkv, hd, page_size, window, [(cached tokens, new rows), ...]
    (9, 3, 64, 16, None, [(0, 200), (0, 64), (0, 1), (0, 65)]),
    (9, 3, 64, 16, None, [(100, 31), (640, 2), (63, 130), (1, 1)]),       # portions that continue a cache
    (4, 4, 64, 32, 100, [(0, 300), (250, 77)]),
    (2, 1, 128, 16, None, [(0, 150), (129, 64)]),
    (6, 2, 128, 64, 37, [(0, 90), (500, 3)]),
]


PREFILL_TC_CASES = [  # the tcgen05 kernel: 128-row query tiles over 128-key tiles, head size 64
    (9, 3, 64, 16, None, [(0, 200), (0, 64), (0, 1), (0, 65)]),
    (9, 3, 64, 16, None, [(100, 31), (640, 2), (63, 130), (1, 1)]),       # portions that continue a cache
    (4, 4, 64, 32, 100, [(0, 300), (250, 77)]),
    (3, 1, 64, 8, None, [(0, 700), (300, 513), (127, 129)]),              # many key tiles, every parity of the rings
    (2, 2, 64, 128, 300, [(0, 1000), (990, 40)]),                         # a page is a whole key tile; a window over tiles
    (5, 5, 64, 64, 5, [(0, 260), (1000, 7)]),
]


def _run_prefill(fn, case):
    from glassbox_b200 import kernels  # noqa: F401
    nh, nkv, hd, ps, window, seqs = case
    dtype = torch.bfloat16
    lens = [c + n for c, n in seqs]
    k, v, tables, dense = make_cache(dtype, len(lens), lens, nkv, hd, ps, seed=4)
    first, row_seq, positions = [0], [], []
    for s_i, (c, n) in enumerate(seqs):
        row_seq += [s_i] * n
        positions += list(range(c, c + n))
        first.append(first[-1] + n)
    n = len(row_seq)
    q = torch.randn(n, nh, hd).to(dtype)
    wide = torch.zeros(n, nh * hd + 2 * nkv * hd, dtype=dtype)               # q sits inside a wider qkv buffer
    wide[:, :nh * hd] = q.reshape(n, -1)
    wide = wide.to(DEV)
    out = torch.full((n, nh * hd), 7.0, device=DEV, dtype=dtype)
    st = status()
    fn(wide[:, :nh * hd], out, k, v, tables, torch.tensor(first, dtype=torch.int32, device=DEV),
       torch.tensor([c for c, _ in seqs], dtype=torch.int32, device=DEV), max(nn for _, nn in seqs),
       nh, nkv, hd, ps, hd ** -0.5, window, st)
    ref = ref_attention(q, dense, row_seq, positions, nh, nkv, hd ** -0.5, window)
    assert int(st) == 0
    diff = (out.cpu().double().reshape(n, nh, hd) - ref).abs()
    worst = int(diff.amax(dim=(1, 2)).argmax())
    assert diff.max() <= tol(dtype, 2), f"row {worst} (sequence, position) = {row_seq[worst], positions[worst]}"


@pytest.mark.parametrize("case", PREFILL_TC_CASES)
def test_attention_prefill_tcgen05(case):
    from glassbox_b200 import kernels
    nh, nkv, hd, ps = case[:4]
    probe = torch.empty(1, nh * hd, device=DEV, dtype=torch.bfloat16)
    assert kernels.attention_prefill_tc_supported(probe, probe, nh, nkv, hd, ps)
    _run_prefill(kernels.attention_prefill_tc, case)


def test_attention_prefill_tcgen05_each_row_finds_its_own_far_key():
    """As the test of the same name below, for the tcgen05 kernel: every query row matches exactly one key
    somewhere before it, on every side of the 128-key tile and page edges."""
    from glassbox_b200 import kernels
    nh, nkv, hd, ps, dtype, L = 2, 1, 64, 16, torch.bfloat16, 530
    k, v, tables, dense = make_cache(dtype, 1, [L], nkv, hd, ps, seed=8)
    kk, vv = dense[0]
    gen = torch.Generator().manual_seed(0)
    targets = [[int(torch.randint(0, p + 1, (1,), generator=gen)) for _ in range(nh)] for p in range(L)]
    q = torch.zeros(L, nh, hd)
    for p in range(L):
        for h in range(nh):
            key = kk[0, targets[p][h]]
            q[p, h] = (key / key.norm() ** 2 * 60.0 * 8.0).float()
    q = q.to(dtype)
    out = torch.empty(L, nh * hd, device=DEV, dtype=dtype)
    st = status()
    kernels.attention_prefill_tc(q.to(DEV).reshape(L, -1), out, k, v, tables, torch.tensor([0, L], dtype=torch.int32, device=DEV),
                                 torch.zeros(1, dtype=torch.int32, device=DEV), L, nh, nkv, hd, ps, hd ** -0.5, None, st)
    assert int(st) == 0
    ref = ref_attention(q, dense, [0] * L, list(range(L)), nh, nkv, hd ** -0.5, None)
    diff = (out.cpu().double().reshape(L, nh, hd) - ref).abs().amax(dim=(1, 2))
    assert diff.max() <= tol(dtype, 2), f"position {int(diff.argmax())} (target {targets[int(diff.argmax())]})"


@pytest.mark.parametrize("case", PREFILL_CASES)
def test_attention_prefill(case):
    from glassbox_b200 import kernels
    nh, nkv, hd, ps, window, seqs = case
    dtype = torch.bfloat16
    assert kernels.attention_prefill_supported(dtype, nh, nkv, hd, ps)
    lens = [c + n for c, n in seqs]
    k, v, tables, dense = make_cache(dtype, len(lens), lens, nkv, hd, ps, seed=4)
    first, row_seq, positions = [0], [], []
    for s_i, (c, n) in enumerate(seqs):
        row_seq += [s_i] * n
        positions += list(range(c, c + n))
        first.append(first[-1] + n)
    n = len(row_seq)
    q = torch.randn(n, nh, hd).to(dtype)
    wide = torch.zeros(n, nh * hd + 2 * nkv * hd, dtype=dtype)               # q sits inside a wider qkv buffer
    wide[:, :nh * hd] = q.reshape(n, -1)
    wide = wide.to(DEV)
    out = torch.full((n, nh * hd), 7.0, device=DEV, dtype=dtype)
    st = status()
    kernels.attention_prefill(wide[:, :nh * hd], out, k, v, tables, torch.tensor(first, dtype=torch.int32, device=DEV),
                              torch.tensor([c for c, _ in seqs], dtype=torch.int32, device=DEV), max(nn for _, nn in seqs),
                              nh, nkv, hd, ps, hd ** -0.5, window, st)
    ref = ref_attention(q, dense, row_seq, positions, nh, nkv, hd ** -0.5, window)
    assert int(st) == 0
    diff = (out.cpu().double().reshape(n, nh, hd) - ref).abs()
    assert diff.max() <= tol(dtype, 2), f"row {int(diff.amax(dim=(1, 2)).argmax())} (sequence, position) = " \
        f"{row_seq[int(diff.amax(dim=(1, 2)).argmax())], positions[int(diff.amax(dim=(1, 2)).argmax())]}"


def test_attention_prefill_each_row_finds_its_own_far_key():
    """Every query row is built to match exactly one key somewhere before it (score 60 above the rest):
    the output must be that key's value, for rows and keys on every side of tile and page edges."""
    from glassbox_b200 import kernels
    nh, nkv, hd, ps, dtype, L = 2, 1, 64, 16, torch.bfloat16, 330
    k, v, tables, dense = make_cache(dtype, 1, [L], nkv, hd, ps, seed=8)
    kk, vv = dense[0]
    gen = torch.Generator().manual_seed(0)
    targets = [[int(torch.randint(0, p + 1, (1,), generator=gen)) for _ in range(nh)] for p in range(L)]
    q = torch.zeros(L, nh, hd)
    for p in range(L):
        for h in range(nh):
            key = kk[0, targets[p][h]]
            q[p, h] = (key / key.norm() ** 2 * 60.0 * 8.0).float()
    q = q.to(dtype)
    out = torch.empty(L, nh * hd, device=DEV, dtype=dtype)
    kernels.attention_prefill(q.to(DEV).reshape(L, -1), out, k, v, tables, torch.tensor([0, L], dtype=torch.int32, device=DEV),
                              torch.zeros(1, dtype=torch.int32, device=DEV), L, nh, nkv, hd, ps, hd ** -0.5, None, status())
    ref = ref_attention(q, dense, [0] * L, list(range(L)), nh, nkv, hd ** -0.5, None)
    diff = (out.cpu().double().reshape(L, nh, hd) - ref).abs().amax(dim=(1, 2))
    assert diff.max() <= tol(dtype, 2), f"position {int(diff.argmax())} (target {targets[int(diff.argmax())]})"


@pytest.mark.parametrize("M", [1, 8, 23, 64])
@pytest.mark.parametrize("N, K", [(576, 576), (100, 264), (3072, 1544), (960, 2560)])
def test_gemm_stream_with_the_norm_folded_in(M, N, K):
    from glassbox_b200 import kernels
    x = torch.randn(M, K, device=DEV) * 3
    gain = 1 + 0.1 * torch.randn(K, device=DEV)
    w = (torch.randn(N, K, device=DEV) / math.sqrt(K)).to(torch.bfloat16)
    h = torch.empty(M, K, device=DEV, dtype=torch.bfloat16)
    kernels.rmsnorm(x, gain, h, 1e-5)
    want = torch.empty(M, N, device=DEV)
    kernels.gemm_stream(h, w, want)                           # the two-kernel way
    got = torch.empty(M, N, device=DEV)
    assert kernels.gemm_stream_supported(x, w)
    kernels.gemm_stream(x, w, got, norm=(gain, 1e-5))         # the folded way
    xd = x.double()
    ref = (gain.double() * (xd / torch.sqrt((xd * xd).mean(-1, keepdim=True) + 1e-5))) @ w.double().T
    assert (got.double() - ref).abs().max() <= tol(torch.bfloat16, 2)
    assert (got - want).abs().max() <= tol(torch.bfloat16, 1)   # same roundings up to the order of one sum


@pytest.mark.parametrize("M", [1, 5, 8, 33, 64])
@pytest.mark.parametrize("nh, nkv, hd, d, ps, rotary", [(9, 3, 64, 576, 16, True), (2, 1, 32, 96, 32, True), (4, 4, 128, 256, 16, False),
                                                          (3, 1, 64, 2048, 16, True)])
def test_gemm_stream_qkv_with_norm_rotary_and_cache_write(M, nh, nkv, hd, d, ps, rotary):
    from glassbox_b200 import kernels
    from glassbox_b200.parts.rope import rotary_table
    dtype = torch.bfloat16
    g = torch.Generator().manual_seed(M)
    x = (torch.randn(M, d, generator=g) * 2).to(DEV)
    gain = (1 + 0.1 * torch.randn(d, generator=g)).to(DEV)
    w = (torch.randn((nh + 2 * nkv) * hd, d, generator=g) / math.sqrt(d)).to(dtype).to(DEV)
    table = rotary_table(1e5, hd, 400).to(DEV) if rotary else None
    positions = torch.randint(0, 400, (M,), generator=g).to(torch.int32)
    pages = 12
    slots = torch.randperm(pages * ps, generator=g)[:M].to(torch.int32)
    if M > 2:
        positions[1] = -1                                  # a padding row: nothing may be stored for it
    # the separate kernels
    h = torch.empty(M, d, device=DEV, dtype=dtype)
    kernels.rmsnorm(x, gain, h, 1e-6)
    qkv = torch.empty(M, (nh + 2 * nkv) * hd, device=DEV, dtype=dtype)
    kernels.gemm_stream(h, w, qkv)
    kc = torch.zeros(pages, nkv, ps, hd, device=DEV, dtype=dtype)
    vc = torch.zeros_like(kc)
    st = status()
    kernels.rope_kv_write(qkv, table, positions.to(DEV), slots.to(DEV), kc, vc, nh, nkv, hd, hd, ps, True, st)
    # the one kernel
    q2 = torch.zeros(M, (nh + 2 * nkv) * hd, device=DEV, dtype=dtype)
    kc2, vc2 = torch.zeros_like(kc), torch.zeros_like(vc)
    # (the kernel takes up to 64 rows; the engine gives it more than 16 only where the rows go in groups of eight)
    assert kernels.gemm_stream_qkv_supported(x, w, hd, q2) == kernels.stream_folds(M, w)
    kernels.gemm_stream_qkv(x, w, q2, table, positions.to(DEV), slots.to(DEV), kc2, vc2, nh, nkv, hd, ps, True, st,
                            norm=(gain, 1e-6))
    assert int(st) == 0
    live = positions >= 0
    t = tol(dtype, 2)
    # a plain float64 statement of the whole operation: normalise, project, rotate the two halves of each head
    xd, wd = x.cpu().double(), w.cpu().double()
    hn = (gain.cpu().double() * (xd / torch.sqrt((xd * xd).mean(dim=1, keepdim=True) + 1e-6))).to(dtype).double()
    ref = (hn @ wd.T).reshape(M, nh + 2 * nkv, hd)
    if rotary:
        cs = table.cpu().double()[positions.clamp(min=0).long()]            # [M, hd/2, 2]
        c, sn = cs[:, None, :, 0], cs[:, None, :, 1]
        rot = ref[:, :nh + nkv].clone()
        a0, a1 = rot[..., :hd // 2].clone(), rot[..., hd // 2:].clone()
        rot[..., :hd // 2], rot[..., hd // 2:] = a0 * c - a1 * sn, a1 * c + a0 * sn
        ref[:, :nh + nkv] = rot
    got_q = q2[:, :nh * hd].cpu().double().reshape(M, nh, hd)
    assert (got_q[live] - ref[live, :nh]).abs().max() <= t, "queries against the float64 statement"
    for r in torch.nonzero(live).flatten().tolist():
        page, offs = int(slots[r]) // ps, int(slots[r]) % ps
        assert (kc2[page, :, offs].cpu().double() - ref[r, nh:nh + nkv]).abs().max() <= t, "keys against the float64 statement"
        assert (vc2[page, :, offs].cpu().double() - ref[r, nh + nkv:]).abs().max() <= t, "values against the float64 statement"
    assert (q2[live.to(DEV), :nh * hd].float() - qkv[live.to(DEV), :nh * hd].float()).abs().max() <= t
    assert (kc2.float() - kc.float()).abs().max() <= t and (vc2.float() - vc.float()).abs().max() <= t
    assert float(q2[~live.to(DEV)].abs().max() if (~live).any() else 0.0) == 0.0
    written = kc2.abs().sum(dim=(1, 3)).flatten().nonzero().numel()     # (page, offset) rows touched
    assert written == int(live.sum())
    # write_kv off: queries only
    kc3, vc3 = torch.zeros_like(kc), torch.zeros_like(vc)
    kernels.gemm_stream_qkv(x, w, q2, table, positions.to(DEV), slots.to(DEV), kc3, vc3, nh, nkv, hd, ps, False, st,
                            norm=(gain, 1e-6))
    assert float(kc3.abs().max()) == 0.0 and float(vc3.abs().max()) == 0.0


@pytest.mark.parametrize("M", [65, 128, 300, 2048])
@pytest.mark.parametrize("nh, nkv, hd, d, ps, rotary", [(9, 3, 64, 576, 16, True), (3, 1, 128, 264, 32, True), (4, 4, 64, 256, 16, False),
                                                          (1, 1, 64, 64, 8, True)])
def test_gemm_tcgen05_qkv_with_rotary_and_cache_write(M, nh, nkv, hd, d, ps, rotary):
    """The tile kernel's QKV epilogue against the separate kernels (product, then rotation and cache write)."""
    from glassbox_b200 import kernels
    from glassbox_b200.parts.rope import rotary_table
    dtype = torch.bfloat16
    g = torch.Generator().manual_seed(M + hd)
    h = torch.randn(M, d, generator=g).to(dtype).to(DEV)
    w = (torch.randn((nh + 2 * nkv) * hd, d, generator=g) / math.sqrt(d)).to(dtype).to(DEV)
    table = rotary_table(1e5, hd, 3000).to(DEV) if rotary else None
    positions = torch.randint(0, 3000, (M,), generator=g).to(torch.int32)
    pages = -(-M // ps) + 3
    slots = torch.randperm(pages * ps, generator=g)[:M].to(torch.int32)
    positions[1] = -1                                      # a padding row: nothing may be stored for it
    qkv = torch.empty(M, (nh + 2 * nkv) * hd, device=DEV, dtype=dtype)
    st = status()
    kernels.gemm_tc(h, w, qkv, status=st)
    kc = torch.zeros(pages, nkv, ps, hd, device=DEV, dtype=dtype)
    vc = torch.zeros_like(kc)
    kernels.rope_kv_write(qkv, table, positions.to(DEV), slots.to(DEV), kc, vc, nh, nkv, hd, hd, ps, True, st)
    q2 = torch.zeros(M, (nh + 2 * nkv) * hd, device=DEV, dtype=dtype)
    kc2, vc2 = torch.zeros_like(kc), torch.zeros_like(vc)
    assert kernels.gemm_tc_qkv_supported(h, w, hd, q2, kc2)
    kernels.gemm_tc_qkv(h, w, q2, table, positions.to(DEV), slots.to(DEV), kc2, vc2, nh, nkv, hd, ps, True, st)
    assert int(st) == 0
    live = (positions >= 0).to(DEV)
    t = tol(dtype, 2)
    assert (q2[live, :nh * hd].float() - qkv[live, :nh * hd].float()).abs().max() <= t
    assert (kc2.float() - kc.float()).abs().max() <= t and (vc2.float() - vc.float()).abs().max() <= t
    assert float(q2[~live].abs().max()) == 0.0 and float(q2[:, nh * hd:].abs().max()) == 0.0   # nothing beside the queries
    written = kc2.abs().sum(dim=(1, 3)).flatten().nonzero().numel()     # (page, offset) rows touched
    assert written == int(live.sum())
    # and against float64: the rotation of the float32 sums
    ref = h.double() @ w.double().T
    if rotary:
        half = hd // 2
        cs = table.double().cpu()[positions.clamp(min=0).long()]        # [M, half, 2]
        r = ref.cpu().reshape(M, nh + 2 * nkv, hd).clone()
        a, b = r[:, :nh + nkv, :half].clone(), r[:, :nh + nkv, half:].clone()
        r[:, :nh + nkv, :half] = a * cs[:, None, :, 0] - b * cs[:, None, :, 1]
        r[:, :nh + nkv, half:] = b * cs[:, None, :, 0] + a * cs[:, None, :, 1]
        ref = r.reshape(M, -1)
    else:
        ref = ref.cpu()
    assert (q2.cpu().double()[live.cpu(), :nh * hd] - ref[live.cpu(), :nh * hd]).abs().max() <= tol(dtype, 2)
    kernels.gemm_tc_qkv(h, w, q2, table, positions.to(DEV), slots.to(DEV), torch.zeros_like(kc), vc3 := torch.zeros_like(vc),
                        nh, nkv, hd, ps, False, st)
    assert float(vc3.abs().max()) == 0.0                                   # write_kv off: queries only


@pytest.mark.parametrize("M, inter, K", [(128, 128, 64), (2048, 1536, 576), (300, 176, 72), (65, 8, 8), (1000, 2560, 960),
                                         (129, 136, 200), (40, 2048, 1024)])
def test_gemm_tcgen05_gated(M, inter, K):
    from glassbox_b200 import kernels
    a = torch.randn(M, K, device=DEV).to(torch.bfloat16)
    w = (torch.randn(2 * inter, K, device=DEV) * (1.5 / math.sqrt(K))).to(torch.bfloat16)
    act = torch.full((M, inter + 3), 9.0, device=DEV, dtype=torch.bfloat16)
    st = status()
    kernels.gemm_tc_gated(a, w, act[:, :inter], status=st)
    assert int(st) == 0, "a bounded wait inside the kernel gave up"
    gu = a.double() @ w.double().T
    g, u = gu[:, :inter], gu[:, inter:]
    ref = g / (1 + torch.exp(-g)) * u
    assert ((act[:, :inter].double() - ref).abs() / (1 + ref.abs())).max() <= tol(torch.bfloat16, 1)
    assert float((act[:, inter:].float() - 9.0).abs().max()) == 0.0        # nothing written beside the output


@pytest.mark.parametrize("M, d, inner, eps", [(65, 576, 1536, 1e-5), (2048, 576, 576, 1e-5), (300, 960, 2560, 1e-6),
                                              (1000, 2048, 512, 1e-5), (129, 72, 200, 1e-3), (4500, 576, 64, 1e-5)])
def test_gemm_tcgen05_norm_split_between_two_products(M, d, inner, eps):
    """An RMSNorm split between the product that completes the residual rows (it also leaves bfloat16(x * gain) and
    partial sums of squares) and the products that read the normalised rows (they scale their sums row by row):
    every output against the float64 statement of add, normalise, multiply."""
    from glassbox_b200 import kernels
    g = torch.Generator().manual_seed(M + d)
    a = torch.randn(M, inner, generator=g).to(torch.bfloat16).to(DEV)
    w = (torch.randn(d, inner, generator=g) / math.sqrt(inner)).to(torch.bfloat16).to(DEV)
    base = (torch.randn(M, d, generator=g) * torch.rand(M, 1, generator=g) * 30).to(DEV)    # rows of very different size
    gain = (1 + 0.3 * torch.randn(d, generator=g)).to(DEV)
    st = status()
    x = base.clone()
    parts = kernels.gemm_tc_column_tiles(M, d, inner)
    pre = torch.full((M, d + 8), 7.0, device=DEV, dtype=torch.bfloat16)
    ss = torch.full((M, parts), -1.0, device=DEV)
    kernels.gemm_tc(a, w, x, accumulate=True, status=st, prepare=(gain, pre[:, :d], ss))
    assert int(st) == 0
    x64 = base.double() + a.double() @ w.double().T
    assert (x.double() - x64).abs().max() <= 2e-5 * math.sqrt(inner) * 30 + 1e-6
    plain = base.clone()
    kernels.gemm_tc(a, w, plain, accumulate=True, status=st)
    assert torch.equal(plain, x), "preparing the norm must not change the residual"
    want_pre = x.double() * gain.double()
    assert ((pre[:, :d].double() - want_pre).abs() / (1e-3 + want_pre.abs())).max() <= 2 ** -8
    assert float((pre[:, d:].float() - 7.0).abs().max()) == 0.0
    sums = (x.double() ** 2).sum(1)
    assert ((ss.double().sum(1) - sums).abs() / sums).max() <= 1e-5
    inv = 1.0 / torch.sqrt(sums / d + eps)
    normed = pre[:, :d].double() * inv[:, None]               # what the consumers see, in exact arithmetic
    scale = kernels.RowScale(ss, eps)
    # plain consumer, float32 and bfloat16 outputs, and one that adds
    n_out = 200
    w2 = (torch.randn(n_out, d, generator=g) / math.sqrt(d)).to(torch.bfloat16).to(DEV)
    ref = normed @ w2.double().T
    c32 = torch.empty(M, n_out, device=DEV)
    kernels.gemm_tc(pre[:, :d], w2, c32, status=st, row_scale=scale)
    assert (c32.double() - ref).abs().max() <= 2e-5 * math.sqrt(d) * float(gain.abs().max()) + 1e-6
    other = torch.randn(M, n_out, generator=g).to(DEV)
    acc = other.clone()
    kernels.gemm_tc(pre[:, :d], w2, acc, accumulate=True, status=st, row_scale=scale)
    assert (acc.double() - other.double() - ref).abs().max() <= 2e-5 * math.sqrt(d) * float(gain.abs().max()) + 1e-6
    # and against the norm as its own kernel in front of the same product
    h = torch.empty(M, d, device=DEV, dtype=torch.bfloat16)
    kernels.rmsnorm(x, gain, h, eps)
    sep = torch.empty(M, n_out, device=DEV)
    kernels.gemm_tc(h, w2, sep, status=st)
    assert (sep - c32).abs().max() <= tol(torch.bfloat16, 2)
    # gated consumer
    inter = 136
    wg = (torch.randn(2 * inter, d, generator=g) * (1.5 / math.sqrt(d))).to(torch.bfloat16).to(DEV)
    act = torch.empty(M, inter, device=DEV, dtype=torch.bfloat16)
    kernels.gemm_tc_gated(pre[:, :d], wg, act, status=st, row_scale=scale)
    gu = normed @ wg.double().T
    gg, uu = gu[:, :inter], gu[:, inter:]
    ref_act = gg / (1 + torch.exp(-gg)) * uu
    assert ((act.double() - ref_act).abs() / (1 + ref_act.abs())).max() <= tol(torch.bfloat16, 1)
    assert int(st) == 0


@pytest.mark.parametrize("M", [65, 300, 2048])
def test_gemm_tcgen05_qkv_completes_a_prepared_norm(M):
    """The QKV epilogue with a row scale: rotation and cache write of inv_rms * (pre W^T), against float64."""
    from glassbox_b200 import kernels
    from glassbox_b200.parts.rope import rotary_table
    nh, nkv, hd, d, ps, eps = 9, 3, 64, 576, 16, 1e-5
    g = torch.Generator().manual_seed(M)
    pre = (torch.randn(M, d, generator=g) * 4).to(torch.bfloat16).to(DEV)
    parts = 3
    ss = (torch.rand(M, parts, generator=g) * d * 20).to(DEV)
    w = (torch.randn((nh + 2 * nkv) * hd, d, generator=g) / math.sqrt(d)).to(torch.bfloat16).to(DEV)
    table = rotary_table(1e5, hd, 3000).to(DEV)
    positions = torch.randint(0, 3000, (M,), generator=g).to(torch.int32)
    pages = -(-M // ps) + 3
    slots = torch.randperm(pages * ps, generator=g)[:M].to(torch.int32)
    q = torch.zeros(M, (nh + 2 * nkv) * hd, device=DEV, dtype=torch.bfloat16)
    kc = torch.zeros(pages, nkv, ps, hd, device=DEV, dtype=torch.bfloat16)
    vc = torch.zeros_like(kc)
    st = status()
    kernels.gemm_tc_qkv(pre, w, q, table, positions.to(DEV), slots.to(DEV), kc, vc, nh, nkv, hd, ps, True, st,
                        row_scale=kernels.RowScale(ss, eps))
    assert int(st) == 0
    inv = 1.0 / torch.sqrt(ss.double().sum(1) / d + eps)
    ref = ((pre.double() * inv[:, None]) @ w.double().T).cpu()
    half = hd // 2
    cs = table.double().cpu()[positions.long()]
    r = ref.reshape(M, nh + 2 * nkv, hd).clone()
    a, b = r[:, :nh + nkv, :half].clone(), r[:, :nh + nkv, half:].clone()
    r[:, :nh + nkv, :half] = a * cs[:, None, :, 0] - b * cs[:, None, :, 1]
    r[:, :nh + nkv, half:] = b * cs[:, None, :, 0] + a * cs[:, None, :, 1]
    t = tol(torch.bfloat16, 2)
    assert (q.cpu().double()[:, :nh * hd] - r[:, :nh].reshape(M, -1)).abs().max() <= t
    for row in range(0, M, 7):
        page, offs = int(slots[row]) // ps, int(slots[row]) % ps
        assert (kc[page, :, offs].cpu().double() - r[row, nh:nh + nkv]).abs().max() <= t
        assert (vc[page, :, offs].cpu().double() - r[row, nh + nkv:]).abs().max() <= t


def test_gemm_tcgen05_many_tiles_per_block():
    """More tiles than SMs: every persistent block walks several tiles and both accumulators alternate."""
    from glassbox_b200 import kernels
    M, N, K = 4096, 4096, 256
    a = torch.randn(M, K, device=DEV).to(torch.bfloat16)
    w = (torch.randn(N, K, device=DEV) / math.sqrt(K)).to(torch.bfloat16)
    c = torch.empty(M, N, device=DEV, dtype=torch.bfloat16)
    st = status()
    kernels.gemm_tc(a, w, c, status=st)
    assert int(st) == 0
    ref = (a.float() @ w.float().T)
    assert (c.float() - ref).abs().max() <= tol(torch.bfloat16, 2)
    base = torch.randn(M, N, device=DEV)
    acc = base.clone()
    kernels.gemm_tc(a, w, acc, accumulate=True, status=st)
    assert (acc - base - ref).abs().max() <= 1e-3 and int(st) == 0


@pytest.mark.parametrize("dtype", DTYPES)
def test_a_position_beyond_the_block_table_is_reported_and_reads_nothing(dtype):
    """The exported launchers take positions and a block table of a stated width from the caller. A position that the
    table does not reach sets the status word and its row comes back as zeros; the rows beside it are served."""
    from glassbox_b200 import kernels
    nh, nkv, hd, ps = 4, 2, 64, 16
    k, v, tables, dense = make_cache(dtype, 2, [40, 40], nkv, hd, ps, extra_pages=0)
    width = tables.shape[1]                                   # 4 pages: positions up to 63
    q = torch.randn(2, nh, hd).to(dtype)
    qd = q.to(DEV).reshape(2, nh * hd)
    row_seq = torch.tensor([0, 1], dtype=torch.int32, device=DEV)
    positions = torch.tensor([39, width * ps + 5], dtype=torch.int32, device=DEV)
    ref = ref_attention(q[:1], dense, [0], [39], nh, nkv, hd ** -0.5, None)

    def check(out, st):
        assert int(st) == 4, "the status word must carry the bad-position bit, and only it"
        got = out.cpu().double().reshape(2, nh, hd)
        assert (got[0] - ref[0]).abs().max() <= tol(dtype, 2) and float(got[1].abs().max()) == 0.0

    st, out = status(), torch.full((2, nh * hd), 7.0, device=DEV, dtype=dtype)
    kernels.attention_rows(qd, out, k, v, tables, row_seq, positions, nh, nkv, hd, ps, hd ** -0.5, None, st)
    check(out, st)
    st, out = status(), torch.full((2, nh * hd), 7.0, device=DEV, dtype=dtype)
    splits = 2
    kernels.attention_decode(qd, out, k, v, tables, row_seq, positions, nh, nkv, hd, ps, hd ** -0.5, None, splits,
                             torch.empty(2 * nh * splits * hd, device=DEV), torch.empty(2 * nh * splits * 2, device=DEV),
                             torch.zeros(2 * nh, dtype=torch.int32, device=DEV), st)
    check(out, st)
    if dtype == torch.bfloat16:
        st, out = status(), torch.full((2, nh * hd), 7.0, device=DEV, dtype=dtype)
        kernels.attention_decode_mma(qd, out, k, v, tables, row_seq, positions, nh, nkv, hd, ps, hd ** -0.5, None, splits,
                                     torch.empty(2 * nh * 4 * splits * hd, device=DEV),
                                     torch.empty(2 * nh * 4 * splits * 2, device=DEV),
                                     torch.zeros(2 * nkv, dtype=torch.int32, device=DEV), st)
        check(out, st)
        st, out = status(), torch.full((2, nh * hd), 7.0, device=DEV, dtype=dtype)
        kernels.attention_prefill(qd, out, k, v, tables, torch.tensor([0, 1, 2], dtype=torch.int32, device=DEV), positions,
                                  1, nh, nkv, hd, ps, hd ** -0.5, None, st)
        check(out, st)


# ------------------------------------------------------------------- the context lengths that are benchmarked
def long_cache(dtype, lens, nkv, hd, ps, seed=0):
    """Random keys and values for sequences of the given lengths on shuffled pages, made on the GPU; returns the
    cache, the block tables (one spare column) and a function that gathers a sequence's keys/values as float64."""
    g = torch.Generator(device=DEV).manual_seed(seed)
    pages_per = [-(-l // ps) for l in lens]
    num_pages = sum(pages_per) + 3
    perm = torch.randperm(num_pages, generator=g, device=DEV)
    k = torch.randn(num_pages, nkv, ps, hd, generator=g, device=DEV).to(dtype)
    v = torch.randn(num_pages, nkv, ps, hd, generator=g, device=DEV).to(dtype)
    tables = torch.full((len(lens), max(pages_per) + 1), -1, dtype=torch.int32, device=DEV)
    at = 0
    for s, n in enumerate(pages_per):
        tables[s, :n] = perm[at:at + n].int()
        at += n

    def dense(s):
        ids = tables[s, :pages_per[s]].long()
        kk = k[ids].permute(1, 0, 2, 3).reshape(nkv, -1, hd)[:, :lens[s]].double()
        vv = v[ids].permute(1, 0, 2, 3).reshape(nkv, -1, hd)[:, :lens[s]].double()
        return kk, vv
    return k, v, tables, dense


def ref_rows_gpu(q, kk, vv, positions, nh, nkv, scale):
    """softmax(q k^T * scale) v in float64 on the GPU, row r seeing keys 0 .. positions[r]; q [n, nh, hd]."""
    n, group = q.shape[0], nh // nkv
    out = torch.empty(n, nh, q.shape[-1], dtype=torch.float64, device=q.device)
    pos = torch.as_tensor(positions, device=q.device)
    keys = torch.arange(kk.shape[1], device=q.device)
    for h in range(nh):
        s = (q[:, h].double() @ kk[h // group].T) * scale
        s = s.masked_fill(keys[None, :] > pos[:, None], float("-inf"))
        out[:, h] = torch.softmax(s, dim=-1) @ vv[h // group]
    return out


LONG_DECODE = [  # heads, kv heads: the benchmark's three models; every batch size it decodes at; 4,096 and 8,192 keys
    (9, 3, 1), (9, 3, 8), (9, 3, 64), (15, 5, 8), (32, 32, 1), (32, 32, 8),
]


@pytest.mark.parametrize("L", [4096, 8192])
@pytest.mark.parametrize("nh, nkv, B", LONG_DECODE)
@pytest.mark.parametrize("dtype", DTYPES)
def test_decode_attention_at_the_benchmarked_context_lengths(dtype, nh, nkv, B, L):
    """The split counts and kernel variants that the engine's own planner picks for these batches (kernels.decode_mma_plan
    and kernels.decode_splits, with the table width a recorded step has), requests of slightly different lengths, and in
    request 0 one far key that carries the whole softmax: near the start, at a split's edge or near the end."""
    from glassbox_b200 import kernels
    hd, ps = 64, 16
    lens = [L - 37 * i for i in range(B)]
    k, v, tables, dense = long_cache(dtype, lens, nkv, hd, ps, seed=B)
    g = torch.Generator(device=DEV).manual_seed(1)
    q = torch.randn(B, nh, hd, generator=g, device=DEV)
    kk0, vv0 = dense(0)
    fars = [5, L // 2 - 1, L - 3]
    for h in range(min(nh, 3)):                                   # heads 0..2 of request 0 each seek one key
        key = kk0[h // (nh // nkv), fars[h]]
        q[0, h] = (key / key.norm() ** 2 * 60.0 * 8.0).float()
    q = q.to(dtype)
    row_seq = torch.arange(B, dtype=torch.int32, device=DEV)
    positions = torch.tensor([l - 1 for l in lens], dtype=torch.int32, device=DEV)
    ref = torch.stack([ref_rows_gpu(q[s:s + 1], *dense(s), [lens[s] - 1], nh, nkv, hd ** -0.5)[0] for s in range(B)])
    for h in range(min(nh, 3)):
        assert (ref[0, h] - vv0[h // (nh // nkv), fars[h]]).abs().max() < 1e-3, "the crafted score does not dominate"
    qd = q.reshape(B, nh * hd)
    st = status()
    out = torch.full((B, nh * hd), 7.0, device=DEV, dtype=dtype)
    if dtype == torch.bfloat16:
        splits, block_keys, warps = kernels.decode_mma_plan(B, nkv, hd, L)
        for sp, bk, nw in {(splits, block_keys, warps), (1, 0, 4), (max(splits // 2, 1), 16, 4), (3, 16, 4), (3, 0, 8), (1, 0, 8), (2, 16, 8)}:
            kernels.attention_decode_mma(qd, out, k, v, tables, row_seq, positions, nh, nkv, hd, ps, hd ** -0.5, None, sp,
                                         torch.empty(B * nh * nw * sp * hd, device=DEV), torch.empty(B * nh * nw * sp * 2, device=DEV),
                                         torch.zeros(B * nkv, dtype=torch.int32, device=DEV), st, bk, nw)
            diff = (out.double().reshape(B, nh, hd) - ref).abs()
            assert int(st) == 0 and diff.max() <= tol(dtype, 2), f"splits {sp}, {bk or 32}-key variant, {nw} warps: off by {float(diff.max()):.3e}"
            out.fill_(7.0)
    splits = kernels.decode_splits(B, nh, nkv, L)
    for sp in {splits, 1, 3}:
        kernels.attention_decode(qd, out, k, v, tables, row_seq, positions, nh, nkv, hd, ps, hd ** -0.5, None, sp,
                                 torch.empty(B * nh * sp * hd, device=DEV), torch.empty(B * nh * sp * 2, device=DEV),
                                 torch.zeros(B * nh, dtype=torch.int32, device=DEV), st)
        diff = (out.double().reshape(B, nh, hd) - ref).abs()
        assert int(st) == 0 and diff.max() <= tol(dtype, 2), f"FMA decode kernel, splits {sp}: off by {float(diff.max()):.3e}"
        out.fill_(7.0)


def test_decode_attention_with_more_pages_than_a_block_stages():
    """One block that covers more than 1,024 pages reads its page ids from the table as it goes instead of from shared
    memory: 20,000 keys in 16-token pages, unsplit and split in two; one far key carries head 0."""
    from glassbox_b200 import kernels
    nh, nkv, hd, ps, L, dtype = 2, 1, 64, 16, 20000, torch.bfloat16
    k, v, tables, dense = long_cache(dtype, [L], nkv, hd, ps, seed=7)
    kk, vv = dense(0)
    q = torch.randn(1, nh, hd, device=DEV)
    q[0, 0] = (kk[0, 17001] / kk[0, 17001].norm() ** 2 * 60.0 * 8.0).float()
    q = q.to(dtype)
    ref = ref_rows_gpu(q, kk, vv, [L - 1], nh, nkv, hd ** -0.5)
    assert (ref[0, 0] - vv[0, 17001]).abs().max() < 1e-3
    out = torch.empty(1, nh * hd, device=DEV, dtype=dtype)
    for splits in (1, 2):
        st = status()
        kernels.attention_decode_mma(q.reshape(1, -1), out, k, v, tables, torch.zeros(1, dtype=torch.int32, device=DEV),
                                     torch.tensor([L - 1], dtype=torch.int32, device=DEV), nh, nkv, hd, ps, hd ** -0.5, None,
                                     splits, torch.empty(nh * 4 * splits * hd, device=DEV),
                                     torch.empty(nh * 4 * splits * 2, device=DEV), torch.zeros(nkv, dtype=torch.int32, device=DEV), st)
        assert int(st) == 0 and (out.double().reshape(1, nh, hd) - ref).abs().max() <= tol(dtype, 2), f"splits {splits}"


@pytest.mark.parametrize("nh, nkv, ps, start, rows", [(3, 1, 16, 0, 4096), (2, 2, 16, 7900, 292), (1, 1, 32, 0, 8192),
                                                      (9, 3, 16, 4000, 96)])
def test_prefill_attention_at_the_benchmarked_context_lengths(nh, nkv, ps, start, rows):
    """Whole prompts of 4,096 and 8,192 tokens (32 and 64 query tiles) and portions that end at 4,096 and 8,192, through
    the tcgen05 kernel and the mma.sync kernel; every 97th row seeks one far key of its own."""
    from glassbox_b200 import kernels
    hd, dtype, L = 64, torch.bfloat16, start + rows
    k, v, tables, dense = long_cache(dtype, [L], nkv, hd, ps, seed=rows)
    kk, vv = dense(0)
    g = torch.Generator(device=DEV).manual_seed(2)
    q = torch.randn(rows, nh, hd, generator=g, device=DEV)
    seekers = list(range(0, rows, 97))
    targets = [int(torch.randint(0, start + r + 1, (1,), generator=g, device=DEV)) for r in seekers]
    for r, t_ in zip(seekers, targets):
        key = kk[0, t_]
        q[r, 0] = (key / key.norm() ** 2 * 60.0 * 8.0).float()
    q = q.to(dtype)
    positions = list(range(start, L))
    ref = ref_rows_gpu(q, kk, vv, positions, nh, nkv, hd ** -0.5)
    for r, t_ in zip(seekers, targets):
        assert (ref[r, 0] - vv[0, t_]).abs().max() < 1e-3
    qd = q.reshape(rows, nh * hd).contiguous()
    first = torch.tensor([0, rows], dtype=torch.int32, device=DEV)
    start_pos = torch.tensor([start], dtype=torch.int32, device=DEV)
    for name, fn in (("tcgen05", kernels.attention_prefill_tc), ("mma.sync", kernels.attention_prefill)):
        out = torch.full((rows, nh * hd), 7.0, device=DEV, dtype=dtype)
        st = status()
        fn(qd, out, k, v, tables, first, start_pos, rows, nh, nkv, hd, ps, hd ** -0.5, None, st)
        diff = (out.double().reshape(rows, nh, hd) - ref).abs().amax(dim=(1, 2))
        assert int(st) == 0 and diff.max() <= tol(dtype, 2), f"{name}: row {int(diff.argmax())} off by {float(diff.max()):.3e}"


# ---------------------------------------------------------------------------- the persistent decode program
def _decode_chain(M, d, nh, nkv, hd, inter, layers, ps, ctx_len, seed):
    """Operands of a chain of decode operations as a model's layers would issue them (norm + QKV + rotation + cache
    write, attention, O projection into the residual, norm + gate/up + SwiGLU, down projection into the residual),
    for M rows that each continue a request of its own."""
    g = torch.Generator(device=DEV).manual_seed(seed)
    bf = torch.bfloat16
    rnd = lambda *shape, s=0.05: (torch.randn(*shape, generator=g, device=DEV) * s).to(bf)
    lens = [ctx_len - 3 * i for i in range(M)]
    k, v, tables, dense = long_cache(bf, lens, nkv, hd, ps, seed=seed)
    w = [dict(wqkv=rnd((nh + 2 * nkv) * hd, d), wo=rnd(d, nh * hd), wgu=rnd(2 * inter, d), wdown=rnd(d, inter),
              g1=1 + 0.1 * torch.randn(d, generator=g, device=DEV), g2=1 + 0.1 * torch.randn(d, generator=g, device=DEV))
         for _ in range(layers)]
    x0 = torch.randn(M, d, generator=g, device=DEV)
    positions = torch.tensor([l - 1 for l in lens], dtype=torch.int32, device=DEV)
    row_seq = torch.arange(M, dtype=torch.int32, device=DEV)
    slots = torch.tensor([int(tables[s, (l - 1) // ps]) * ps + (l - 1) % ps for s, l in enumerate(lens)], dtype=torch.int32, device=DEV)
    from glassbox_b200.parts.rope import rotary_table
    rope = rotary_table(10000.0, hd, ctx_len + 8).to(DEV)
    return dict(k=k, v=v, tables=tables, w=w, x0=x0, positions=positions, row_seq=row_seq, slots=slots, rope=rope, lens=lens)


def _run_chain(c, M, d, nh, nkv, hd, inter, ps, st, splits):
    from glassbox_b200 import kernels
    bf = torch.bfloat16
    x = c["x0"].clone()
    k, v = c["k"].clone(), c["v"].clone()
    qkv = torch.zeros(M, (nh + 2 * nkv) * hd, device=DEV, dtype=bf)
    att = torch.zeros(M, nh * hd, device=DEV, dtype=bf)
    act = torch.zeros(M, inter, device=DEV, dtype=bf)
    part_acc = torch.empty(M * nh * 4 * splits * hd, device=DEV)
    part_ml = torch.empty(M * nh * 4 * splits * 2, device=DEV)
    counters = torch.zeros(M * nkv, dtype=torch.int32, device=DEV)
    for lw in c["w"]:
        kernels.gemm_stream_qkv(x, lw["wqkv"], qkv, c["rope"], c["positions"], c["slots"], k, v, nh, nkv, hd, ps, True, st,
                                norm=(lw["g1"], 1e-5))
        kernels.attention_decode_mma(qkv[:, :nh * hd], att, k, v, c["tables"], c["row_seq"], c["positions"], nh, nkv, hd, ps,
                                     hd ** -0.5, None, splits, part_acc, part_ml, counters, st)
        kernels.gemm_stream(att, lw["wo"], x, accumulate=True)
        kernels.gemm_stream(x, lw["wgu"], act, gated=True, norm=(lw["g2"], 1e-5))
        kernels.gemm_stream(act, lw["wdown"], x, accumulate=True)
    return x, k, v, (qkv, att, act, part_acc, part_ml, counters)


@pytest.mark.parametrize("how", ["by rows", "by operations"])
@pytest.mark.parametrize("M", [1, 5, 8, 13, 16])
@pytest.mark.parametrize("d, nh, nkv, hd, inter", [(576, 9, 3, 64, 512), (96, 3, 1, 32, 176), (256, 2, 2, 128, 320)])
def test_decode_program_runs_the_operations_the_kernels_would(M, d, nh, nkv, hd, inter, how):
    """The same chain of calls, once launched kernel by kernel and once recorded into a program and run by a
    persistent kernel. Shared by operations, the persistent kernel runs the stand-alone kernels' own bodies: with every K
    below 1,024 those take the same 512-wide chunks and no cluster, so the sums are formed in the same order and the
    results must be equal bit for bit, residual rows and cache alike. Shared by rows, it forms plain dot products.
    Run twice, so that the barrier word and the attention's counters are shown to come back to their start."""
    from glassbox_b200 import kernels
    ps, layers, ctx_len, splits = 16, 3, 300, 3
    c = _decode_chain(M, d, nh, nkv, hd, inter, layers, ps, ctx_len, seed=M)
    st = status()
    want_x, want_k, want_v, _ = _run_chain(c, M, d, nh, nkv, hd, inter, ps, st, splits)
    assert int(st) == 0
    prog = kernels.Program()
    prog.how = kernels.BY_ROWS if how == "by rows" else kernels.BY_OPERATIONS
    for rep in range(2):
        before = kernels.launch_count
        kernels.program_begin(prog, st)
        try:
            got_x, got_k, got_v, keep = _run_chain(c, M, d, nh, nkv, hd, inter, ps, st, splits)
        finally:
            kernels.program_end()
        assert kernels.launch_count - before == 1, "the chain was not one launch"
        assert int(st) == 0
        if how == "by operations":
            assert torch.equal(got_x, want_x) and torch.equal(got_k, want_k) and torch.equal(got_v, want_v), f"pass {rep}"
        else:   # the by-rows kernel adds up in another order (plain dot products): equal within bfloat16 rounding of the chain
            scale = float(want_x.abs().max())
            assert float((got_x - want_x).abs().max()) <= 2e-2 * scale, f"pass {rep}: {float((got_x - want_x).abs().max()):.3e} of {scale:.3e}"
            assert float((got_k.float() - want_k.float()).abs().max()) <= 2e-2 * float(want_k.float().abs().max())
            assert float((got_v.float() - want_v.float()).abs().max()) <= 2e-2 * float(want_v.float().abs().max())
        assert len(prog.segments) == 1
        del keep


@pytest.mark.parametrize("how", ["by rows", "by operations"])
def test_decode_program_with_long_k_and_a_kernel_in_between(how):
    """K of 1,536 and 2,048 (the stand-alone kernel would split these over a cluster: another order of the sums, so the
    comparison is with a float64 statement), and a kernel that is not part of programs in the middle of the chain: what was
    recorded before it must run before it, what comes after it after."""
    from glassbox_b200 import kernels
    M, d, inter = 7, 2048, 1536
    g = torch.Generator(device=DEV).manual_seed(3)
    bf = torch.bfloat16
    a = (torch.randn(M, d, generator=g, device=DEV)).to(bf)
    w1 = (torch.randn(inter * 2, d, generator=g, device=DEV) * 0.03).to(bf)
    w2 = (torch.randn(d, inter, generator=g, device=DEV) * 0.03).to(bf)
    act = torch.zeros(M, inter, device=DEV, dtype=bf)
    acted = torch.zeros(M, inter, device=DEV, dtype=bf)
    x = torch.zeros(M, d, device=DEV)
    gate_up = torch.zeros(M, 2 * inter, device=DEV, dtype=bf)
    prog, st = kernels.Program(), status()
    prog.how = kernels.BY_ROWS if how == "by rows" else kernels.BY_OPERATIONS
    kernels.program_begin(prog, st)
    try:
        kernels.gemm_stream(a, w1, gate_up)                       # recorded
        kernels.swiglu(gate_up, acted)                            # launched: flushes the product before it
        kernels.gemm_stream(a, w1, act, gated=True)               # recorded
        kernels.gemm_stream(act, w2, x, accumulate=True)          # recorded: reads what the one before wrote
    finally:
        kernels.program_end()
    assert len(prog.segments) == 2 and int(st) == 0
    gu = a.double() @ w1.double().T
    ref_act = (gu[:, :inter] / (1 + torch.exp(-gu[:, :inter])) * gu[:, inter:])
    assert (acted.double() - ref_act).abs().max() <= 0.02 * ref_act.abs().max()
    assert torch.equal(act, acted) or (act.double() - acted.double()).abs().max() <= 0.01 * ref_act.abs().max()
    ref_x = act.double() @ w2.double().T
    assert (x.double() - ref_x).abs().max() <= 2e-3 * ref_x.abs().max()


def test_a_wait_at_the_programs_barrier_that_runs_out_is_reported_and_harms_nothing():
    """The persistent kernel's barrier waits are bounded. Here every barrier is told to expect one block more than the
    grid has and to give up after a millisecond of cycles: the kernel must return by itself, the status word must carry
    the wait-timeout bit, the operations behind the first barrier must not have run, and the same program launched
    normally right afterwards must work."""
    from glassbox_b200 import kernels
    M, d = 4, 256
    g = torch.Generator(device=DEV).manual_seed(5)
    a = torch.randn(M, d, generator=g, device=DEV).to(torch.bfloat16)
    w = (torch.randn(d, d, generator=g, device=DEV) * 0.05).to(torch.bfloat16)
    h = torch.zeros(M, d, device=DEV, dtype=torch.bfloat16)
    out = torch.full((M, d), 7.0, device=DEV)

    def chain(prog, st):
        kernels.program_begin(prog, st)
        try:
            kernels.gemm_stream(a, w, h)
            kernels.gemm_stream(h, w, out)
        finally:
            kernels.program_end()

    prog, st = kernels.Program(), status()
    prog.absent_blocks, prog.wait_cycles = 1, 2_000_000
    chain(prog, st)
    torch.cuda.synchronize()
    assert int(st) == 8, "the wait-timeout bit, and only it"
    assert float((out - 7.0).abs().max()) == 0.0, "an operation behind the barrier ran although the barrier never opened"
    with pytest.raises(kernels.KernelError, match="bounded wait"):
        kernels.check_status(st)
    prog.absent_blocks = 0
    chain(prog, st)
    ref = (a.double() @ w.double().T).to(torch.bfloat16).double() @ w.double().T
    assert int(st) == 0 and (out.double() - ref).abs().max() <= 1e-2 * ref.abs().max()
