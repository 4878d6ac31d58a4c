"""Each kernel alone against the plain implementation's function for the same op, at sizes other
than the engine's tiny models: odd widths, head sizes in steps of 16, odd head and group counts."""
import math

import pytest
import torch

from tests.plain import llama_plain as plain

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
DT = [torch.float32, torch.bfloat16]
IDS = ["f32", "bf16"]
# elementwise results: float32 to rounding; bfloat16 outputs are rounded once to 8 bits (2^-9 relative)
ETOL = {torch.float32: 2e-6, torch.bfloat16: 2 ** -8}


def rel(a, b):
    return float((a.double().cpu() - b.double().cpu()).abs().max() / b.double().abs().max().clamp_min(1e-30))


def K():
    from vllm_oxide_b200 import kernels
    return kernels


def test_embed():
    g = torch.Generator().manual_seed(0)
    for dt in DT:
        table = torch.randn(301, 72, generator=g).to(dt).to(DEV)
        toks = torch.tensor([0, 300, 17, 17, 5], dtype=torch.int32, device=DEV)
        out = torch.empty(5, 72, dtype=torch.float32, device=DEV)
        flag = torch.zeros(1, dtype=torch.int32, device=DEV)
        K().embed(table, toks, out, flag)
        want = plain.embedding(table.double().cpu(), toks.tolist())
        assert torch.equal(out.double().cpu(), want) and int(flag) == 0
        bad = torch.tensor([1, 301, 2, 3, 4], dtype=torch.int32, device=DEV)
        K().embed(table, bad, out, flag)
        assert int(flag) == 1 and float(out[1].abs().max()) == 0.0      # out of range: zeros and a raised flag


@pytest.mark.parametrize("dt", DT, ids=IDS)
@pytest.mark.parametrize("h", [19, 100, 2048, 4100])
def test_add_rmsnorm(dt, h):
    g = torch.Generator().manual_seed(h)
    T = 7
    resid = torch.randn(T, h, generator=g).to(DEV)
    delta = (torch.randn(T, h, generator=g) * 0.5).to(dt).to(DEV)
    w = (1 + 0.3 * torch.randn(h, generator=g)).to(DEV)
    eps = 3e-5
    r0 = resid.clone()
    out = torch.empty(T, h, dtype=dt, device=DEV)
    K().add_rmsnorm(resid, delta, w, eps, out)
    x = r0.double().cpu() + delta.double().cpu()
    assert rel(resid, x) <= 2e-7                                       # the residual sum stays float32
    assert rel(out, plain.rms_norm(x, w.double().cpu(), eps)) <= ETOL[dt]
    # without delta, and with a row list: the residual is left alone
    r1 = resid.clone()
    rows = torch.tensor([6, 0, 3], dtype=torch.int32, device=DEV)
    out2 = torch.empty(3, h, dtype=dt, device=DEV)
    K().add_rmsnorm(resid, delta, w, eps, out2, rows)
    assert torch.equal(resid, r1)
    x2 = (r1.double().cpu() + delta.double().cpu())[[6, 0, 3]]
    assert rel(out2, plain.rms_norm(x2, w.double().cpu(), eps)) <= ETOL[dt]
    out3 = torch.empty(T, h, dtype=dt, device=DEV)
    K().add_rmsnorm(resid, None, w, eps, out3)
    assert rel(out3, plain.rms_norm(r1.double().cpu(), w.double().cpu(), eps)) <= ETOL[dt]


def test_rmsnorm_refuses_too_wide_rows():
    from vllm_oxide_b200.errors import ShapeError
    with pytest.raises(ShapeError, match="limit"):
        K().add_rmsnorm(torch.zeros(1, 20000, device=DEV), None, torch.ones(20000, device=DEV), 1e-5,
                        torch.zeros(1, 20000, device=DEV))


@pytest.mark.parametrize("dt", DT, ids=IDS)
@pytest.mark.parametrize("I", [5, 224, 1000])
def test_swiglu(dt, I):
    g = torch.Generator().manual_seed(I)
    gu = (torch.randn(6, 2 * I, generator=g) * 3).to(dt).to(DEV)
    out = torch.empty(6, I, dtype=dt, device=DEV)
    K().swiglu(gu, out)
    want = plain.swiglu(gu[:, :I].double().cpu(), gu[:, I:].double().cpu())
    assert rel(out, want) <= ETOL[dt]


@pytest.mark.parametrize("M,N,K_", [(1, 1, 1), (7, 37, 21), (64, 64, 16), (65, 130, 257), (3, 1000, 96), (200, 50, 2048)])
def test_gemm_f32(M, N, K_):
    # odd sizes against the 64x64x16 tiling (the reference tests 7x21 -> 37: crates/engine/src/backend/cpu/tests.rs:37-59)
    g = torch.Generator().manual_seed(M * 1000 + N)
    a = torch.randn(M, K_, generator=g).to(DEV)
    w = torch.randn(N, K_, generator=g).to(DEV)
    out = torch.empty(M, N, device=DEV)
    K().gemm_f32(a, w, out)
    # one chain of K float32 FMAs per element: rounding errors of 2^-24 each add up like a random
    # walk, sqrt(K) * 2^-24 of the running sum; twice that as the bound (1e-6 at the reference's K = 21)
    tol = max(1e-6, 2.0 ** -23 * math.sqrt(K_))
    assert rel(out, plain.linear(a.double().cpu(), w.double().cpu())) <= tol
    # a row's value does not depend on the rows around it: bitwise
    out1 = torch.empty(1, N, device=DEV)
    K().gemm_f32(a[M - 1:M], w, out1)
    assert torch.equal(out1[0], out[M - 1])
    # strided views (a column slice of a wider buffer)
    wide = torch.randn(M, K_ + 8, generator=g).to(DEV)
    outw = torch.zeros(M, N + 4, device=DEV)
    K().gemm_f32(wide[:, 4:4 + K_], w, outw[:, 2:2 + N])
    assert rel(outw[:, 2:2 + N], plain.linear(wide[:, 4:4 + K_].double().cpu(), w.double().cpu())) <= tol
    assert float(outw[:, :2].abs().max()) == 0.0 and float(outw[:, 2 + N:].abs().max()) == 0.0


def test_gemm_f32_shape_errors():
    from vllm_oxide_b200.errors import ShapeError
    with pytest.raises(ShapeError):
        K().gemm_f32(torch.zeros(2, 3, device=DEV), torch.zeros(4, 5, device=DEV), torch.zeros(2, 4, device=DEV))
    with pytest.raises(ShapeError):
        K().gemm_f32(torch.zeros(2, 3, device=DEV), torch.zeros(4, 3, device=DEV), torch.zeros(2, 5, device=DEV))


def test_linear_bf16_library_product():
    g = torch.Generator().manual_seed(3)
    a = torch.randn(9, 200, generator=g).to(torch.bfloat16).to(DEV)
    w = torch.randn(77, 200, generator=g).to(torch.bfloat16).to(DEV)
    want = plain.linear(a.double().cpu(), w.double().cpu())
    o32 = torch.empty(9, 77, dtype=torch.float32, device=DEV)
    K().linear(a, w, o32)
    assert rel(o32, want) <= 1e-5                                      # bf16 inputs are exact; float32 accumulation
    o16 = torch.empty(9, 77, dtype=torch.bfloat16, device=DEV)
    K().linear(a, w, o16)
    assert rel(o16, want) <= 2 ** -8


def _paged_case(dt, H, KV, hd, page, seqs, seed, scale_key=None, poison=False):
    """seqs: list of (context_len, num_new). Returns tensors for the kernel and per-sequence q/k/v."""
    g = torch.Generator().manual_seed(seed)
    total_pages = sum(-(-(c + n) // page) for c, n in seqs) + 3
    perm = torch.randperm(total_pages, generator=g).tolist()          # shuffled, non-identity tables
    kc = torch.randn(total_pages, KV, page, hd, generator=g).to(dt)   # stale values everywhere
    vc = torch.randn(total_pages, KV, page, hd, generator=g).to(dt)
    if poison:                                                        # what no request wrote is NaN: it must reach no result
        kc.fill_(float("nan"))
        vc.fill_(float("nan"))
    max_pages = max(-(-(c + n) // page) for c, n in seqs) + 1
    bt = torch.full((len(seqs), max_pages), -1, dtype=torch.int32)
    qs, ks, vs, row_seq, positions = [], [], [], [], []
    for s, (c, n) in enumerate(seqs):
        L = c + n
        k = torch.randn(L, KV * hd, generator=g).to(dt)
        v = torch.randn(L, KV * hd, generator=g).to(dt)
        q = torch.randn(L, H * hd, generator=g).to(dt)
        if scale_key is not None:
            j = scale_key(L)
            k[j] *= 6.0                       # one key stands out: a wrong or missing key shows
        np_ = -(-L // page)
        for i in range(np_):
            bt[s, i] = perm.pop()
        for p in range(L):
            pg, off = int(bt[s, p // page]), p % page
            kc[pg, :, off, :] = k[p].view(KV, hd)
            vc[pg, :, off, :] = v[p].view(KV, hd)
        qs.append(q), ks.append(k), vs.append(v)
        row_seq += [s] * n
        positions += list(range(c, L))
    qrows = torch.cat([q[c:] for q, (c, n) in zip(qs, seqs)])
    return (qrows, kc, vc, bt, torch.tensor(row_seq, dtype=torch.int32), torch.tensor(positions, dtype=torch.int32),
            qs, ks, vs)


ATOL = {torch.float32: 1e-5, torch.bfloat16: 2 ** -7}      # reference: 1e-5 relative for paged attention (cpu/tests.rs:161-334)


@pytest.mark.parametrize("dt", DT, ids=IDS)
@pytest.mark.parametrize("H,KV,hd,page", [(6, 2, 16, 4), (3, 1, 32, 8), (5, 5, 48, 16), (8, 2, 64, 16), (4, 2, 128, 16),
                                          (2, 1, 256, 32), (7, 7, 80, 8)])
def test_paged_attention_prefill_and_decode_shapes(dt, H, KV, hd, page):
    # (context, new): mid-page, zero context, page edge, a decode row, a long one
    seqs = [(5, 6), (0, 3), (2 * page, page), (37, 1), (0, 1), (3 * page - 1, 2)]
    qrows, kc, vc, bt, row_seq, pos, qs, ks, vs = _paged_case(dt, H, KV, hd, page, seqs, seed=hd + H)
    out = torch.empty_like(qrows).to(DEV)
    K().paged_attention(qrows.to(DEV), out, kc.to(DEV), vc.to(DEV), bt.to(DEV), row_seq.to(DEV), pos.to(DEV),
                        H, KV, hd, 1.0 / math.sqrt(hd))
    r = 0
    for s, (c, n) in enumerate(seqs):
        want = plain.causal_attention(qs[s].double(), ks[s].double(), vs[s].double(), H, KV, hd)[c:]
        got = out[r:r + n]
        assert rel(got, want) <= ATOL[dt], (s, c, n)
        r += n


@pytest.mark.parametrize("dt", DT, ids=IDS)
def test_paged_attention_far_key_among_hundreds(dt):
    """One key far back dominates the softmax; it must be found at any distance, across pages."""
    H, KV, hd, page = 4, 2, 64, 16
    seqs = [(700, 1), (0, 333), (511, 2)]
    qrows, kc, vc, bt, row_seq, pos, qs, ks, vs = _paged_case(dt, H, KV, hd, page, seqs, seed=1, scale_key=lambda L: 3)
    out = torch.empty_like(qrows).to(DEV)
    K().paged_attention(qrows.to(DEV), out, kc.to(DEV), vc.to(DEV), bt.to(DEV), row_seq.to(DEV), pos.to(DEV),
                        H, KV, hd, 1.0 / math.sqrt(hd))
    r = 0
    for s, (c, n) in enumerate(seqs):
        want = plain.causal_attention(qs[s].double(), ks[s].double(), vs[s].double(), H, KV, hd)[c:]
        assert rel(out[r:r + n], want) <= ATOL[dt]
        r += n


@pytest.mark.parametrize("dt", DT, ids=IDS)
@pytest.mark.parametrize("window", [1, 5, 16, 17, 40])
def test_paged_attention_window_edge(dt, window):
    H, KV, hd, page = 4, 2, 32, 8
    seqs = [(0, 50), (44, 3), (window, 1), (max(window - 1, 0), 1)]
    # the key just outside the window stands out: reading it would change everything
    qrows, kc, vc, bt, row_seq, pos, qs, ks, vs = _paged_case(dt, H, KV, hd, page, seqs, seed=window,
                                                             scale_key=lambda L: max(L - 1 - window, 0))
    out = torch.empty_like(qrows).to(DEV)
    K().paged_attention(qrows.to(DEV), out, kc.to(DEV), vc.to(DEV), bt.to(DEV), row_seq.to(DEV), pos.to(DEV),
                        H, KV, hd, 0.3, window)
    r = 0
    for s, (c, n) in enumerate(seqs):
        want = plain.causal_attention(qs[s].double(), ks[s].double(), vs[s].double(), H, KV, hd, window=window, scale=0.3)[c:]
        assert rel(out[r:r + n], want) <= ATOL[dt]
        r += n


def test_paged_attention_refuses_bad_sizes():
    from vllm_oxide_b200.errors import ShapeError
    q = torch.zeros(1, 4 * 20, device=DEV)
    kc = torch.zeros(2, 2, 8, 20, device=DEV)
    z = torch.zeros(1, dtype=torch.int32, device=DEV)
    with pytest.raises(ShapeError, match="head_dim 20"):
        K().paged_attention(q, q.clone(), kc, kc, torch.zeros(1, 2, dtype=torch.int32, device=DEV), z, z, 4, 2, 20, 1.0)
    q = torch.zeros(1, 3 * 16, device=DEV)
    kc = torch.zeros(2, 2, 8, 16, device=DEV)
    with pytest.raises(ShapeError, match="multiple"):
        K().paged_attention(q, q.clone(), kc, kc, torch.zeros(1, 2, dtype=torch.int32, device=DEV), z, z, 3, 2, 16, 1.0)


@pytest.mark.parametrize("dt", DT, ids=IDS)
@pytest.mark.parametrize("T,pad", [(11, 0), (70, 0), (70, 1)])      # few tokens; many (16-byte accesses); many, rows not 16-byte aligned
@pytest.mark.parametrize("H,KV,hd,page", [(6, 2, 16, 4), (3, 1, 32, 8), (5, 5, 48, 16), (32, 8, 64, 16), (2, 1, 256, 16)])
def test_rope_kv_write(dt, H, KV, hd, page, T, pad):
    g = torch.Generator().manual_seed(hd)
    cfg = {"head_dim": hd, "hidden_size": H * hd, "num_attention_heads": H, "rope_theta": 500000.0,
           "rope_scaling": {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                            "original_max_position_embeddings": 64}}
    inv = plain.rope_inv_freq(cfg)
    qkv = torch.randn(T, (H + 2 * KV) * hd, generator=g).to(dt)
    positions = ([0, 1, 2, 63, 64, 65, 1000, 4095, 7, 7, 300] + list(range(100, 100 + T)))[:T]
    pages = -(-T // page) + 9
    slots = torch.randperm(pages * page, generator=g)[:T].to(torch.int32)
    slots[4] = -1                                                       # this token writes nothing
    kc = torch.full((pages, KV, page, hd), 7.0).to(dt)
    vc = torch.full((pages, KV, page, hd), 7.0).to(dt)
    d_kc, d_vc = kc.to(DEV), vc.to(DEV)
    d_qkv = torch.zeros(T, qkv.shape[1] + pad, dtype=dt, device=DEV)[:, :qkv.shape[1]]
    d_qkv.copy_(qkv)
    q, k, v = d_qkv[:, :H * hd], d_qkv[:, H * hd:(H + KV) * hd], d_qkv[:, (H + KV) * hd:]
    K().rope_kv_write(q, k, v, torch.tensor(positions, dtype=torch.int32, device=DEV), slots.to(DEV), inv.to(DEV),
                      d_kc, d_vc, H, KV, hd)
    wq = plain.rope(qkv[:, :H * hd].double(), positions, inv, hd)
    wk = plain.rope(qkv[:, H * hd:(H + KV) * hd].double(), positions, inv, hd)
    tol = 3e-6 if dt == torch.float32 else 2 ** -8
    assert rel(q, wq) <= tol and rel(k, wk) <= tol
    for t in range(T):
        s = int(slots[t])
        if s < 0:
            continue
        pg, off = s // page, s % page
        assert rel(d_kc[pg, :, off, :].reshape(-1), wk[t]) <= tol
        assert torch.equal(d_vc[pg, :, off, :].reshape(-1).cpu(), qkv[t, (H + KV) * hd:])
    written = {int(s) for s in slots if s >= 0}
    for s in range(pages * page):
        if s not in written:
            assert float((d_kc[s // page, :, s % page, :].float() - 7.0).abs().max()) == 0.0     # nothing else is touched


def test_pick_tokens_greedy_cases():
    # crates/engine/src/backend/cpu/tests.rs:129-144: ties -> first, all equal -> 0, NaN -> error
    V = 10007
    logits = torch.full((5, V), -1.0, device=DEV)
    logits[0, 5000] = 5.0
    logits[0, 9000] = 5.0
    logits[1] = 0.0
    logits[2, V - 1] = 3.0
    logits[3, 0] = 2.0
    logits[4, 77] = float("nan")
    k = K()
    sp = k.pick_splits(V)
    out = torch.zeros(5, dtype=torch.int32, device=DEV)
    flags = torch.zeros(5, dtype=torch.int32, device=DEV)
    k.pick_tokens(logits, out, flags, torch.empty(5 * sp, device=DEV), torch.empty(5 * sp, dtype=torch.int32, device=DEV))
    assert out.tolist() == [5000, 0, V - 1, 0, -1]
    assert flags.tolist() == [0, 0, 0, 0, 0]          # the flag is cleared once it has been turned into -1
    want = [plain.argmax_first(r) for r in logits[:4].double().cpu()]
    assert out.tolist()[:4] == want


def test_pick_writes_its_tokens_to_further_places():
    """`also`: the pick kernel writes the same tokens to up to two more places, a device tensor and a
    page-locked host buffer that the device addresses directly (no copy behind the kernel); both the
    two-pass pick and the final pass alone; what lies around the rows stays as it was."""
    from vllm_oxide_b200.errors import ShapeError
    V = 10007
    logits = torch.full((5, V), -1.0, device=DEV)
    for r, i in enumerate([5000, 3, V - 1, 0, 77]):
        logits[r, i] = 2.0 + r
    logits[4, 78] = float("nan")
    k = K()
    sp = k.pick_splits(V)
    host = k.HostInts((2, 8))
    host.tensor.fill_(-7)
    dev2 = torch.full((9,), -7, dtype=torch.int32, device=DEV)
    out = torch.zeros(5, dtype=torch.int32, device=DEV)
    flags = torch.zeros(5, dtype=torch.int32, device=DEV)
    val, idx = torch.empty(5 * sp, device=DEV), torch.empty(5 * sp, dtype=torch.int32, device=DEV)
    k.pick_tokens(logits, out, flags, val, idx, also=[dev2[2:7], host.at(8 + 1)])
    torch.cuda.synchronize()
    want = [5000, 3, V - 1, 0, -1]
    assert out.tolist() == want and dev2.tolist() == [-7, -7] + want + [-7, -7]
    assert host.tensor.tolist() == [[-7] * 8, [-7] + want + [-7, -7]]
    # the final pass alone, pairs given: one destination only
    part_val = torch.tensor([[1.0, 5.0, 5.0], [0.0, -1.0, 7.0]], device=DEV)
    part_idx = torch.tensor([[9, 4, 6], [1, 2, 3]], dtype=torch.int32, device=DEV)
    out2 = torch.zeros(2, dtype=torch.int32, device=DEV)
    k.pick_final(part_val, part_idx, 2, 100, torch.zeros(2, dtype=torch.int32, device=DEV), out2, also=[host.at(0)])
    torch.cuda.synchronize()
    assert out2.tolist() == [4, 3] and host.tensor[0].tolist() == [4, 3] + [-7] * 6
    with pytest.raises(ShapeError, match="room for"):
        k.pick_final(part_val, part_idx, 2, 100, flags, out2, also=[host.at(15)])
    with pytest.raises(ShapeError, match="at most two"):
        k.pick_final(part_val, part_idx, 2, 100, flags, out2, also=[out2, out2, out2])
    with pytest.raises(ShapeError):
        k.pick_tokens(logits, out, flags, val, idx, also=[dev2[:3]])


def test_pick_tokens_temperature_matches_plain_and_law():
    V = 997
    g = torch.Generator().manual_seed(5)
    logits = (torch.randn(6, V, generator=g) * 2).to(DEV)
    temps = torch.tensor([0.7, 0.0, 1.3, 0.7, 0.7, 0.2], device=DEV)
    seeds = torch.tensor([[1, 0], [2, 0], [3, 7], [1, 0], [9, 1], [4, 4]], dtype=torch.int32, device=DEV)
    steps = torch.tensor([0, 5, 2, 1, 0, 3], dtype=torch.int32, device=DEV)
    k = K()
    sp = k.pick_splits(V)
    out = torch.zeros(6, dtype=torch.int32, device=DEV)
    k.pick_tokens(logits, out, torch.zeros(6, dtype=torch.int32, device=DEV), torch.empty(6 * sp, device=DEV),
                  torch.empty(6 * sp, dtype=torch.int32, device=DEV), temps, seeds, steps)
    for r in range(6):
        seed = (int(seeds[r, 1]) << 32) | int(seeds[r, 0])
        assert int(out[r]) == plain.temperature_pick(logits[r].double().cpu(), float(temps[r]), seed, int(steps[r]))
    # the law: many steps of one request over small logits follow softmax(logits / t)
    small = torch.tensor([[2.0, 1.0, 0.0, -1.0, -30.0]], device=DEV).repeat(64, 1)
    n, counts = 0, torch.zeros(5)
    for it in range(40):
        st = torch.arange(it * 64, it * 64 + 64, dtype=torch.int32, device=DEV)
        o = torch.zeros(64, dtype=torch.int32, device=DEV)
        k.pick_tokens(small, o, torch.zeros(64, dtype=torch.int32, device=DEV), torch.empty(64, device=DEV),
                      torch.empty(64, dtype=torch.int32, device=DEV), torch.full((64,), 0.7, device=DEV),
                      torch.tensor([[11, 3]] * 64, dtype=torch.int32, device=DEV), st)
        counts += torch.bincount(o.cpu(), minlength=5).float()
        n += 64
    p = torch.softmax(small[0].cpu().double() / 0.7, 0)
    for i in range(5):
        assert abs(float(counts[i]) / n - float(p[i])) < 4 * math.sqrt(float(p[i]) * (1 - float(p[i])) / n) + 2e-3


def test_cpu_tensors_are_refused():
    from vllm_oxide_b200.errors import KernelError
    with pytest.raises(KernelError, match="no CPU path"):
        K().gemm_f32(torch.zeros(2, 2), torch.zeros(2, 2), torch.zeros(2, 2))


# ----------------------------------------------------------------------------- tensor-core attention (bfloat16)
def _starts_ctx(seqs):
    starts, ctxs, r = [0], [], 0
    for c, n in seqs:
        r += n
        starts.append(r)
        ctxs.append(c)
    return torch.tensor(starts, dtype=torch.int32, device=DEV), torch.tensor(ctxs, dtype=torch.int32, device=DEV)


@pytest.mark.parametrize("window", [0, 70])
@pytest.mark.parametrize("H,KV,hd,page", [(8, 2, 64, 16), (3, 1, 64, 8), (4, 4, 128, 32), (6, 2, 128, 16), (32, 8, 64, 64)])
def test_attn_prefill_mma(H, KV, hd, page, window):
    dt = torch.bfloat16
    # portions that start mid-page, at a page edge, at zero; single tokens beside them; > one row tile
    seqs = [(5, 6), (0, 3), (2 * page, page), (137, 1), (0, 1), (3 * page - 1, 2), (0, 150), (201, 77)]
    sk = (lambda L: max(L - 1 - window, 0)) if window else (lambda L: min(3, L - 1))
    qrows, kc, vc, bt, row_seq, pos, qs, ks, vs = _paged_case(dt, H, KV, hd, page, seqs, seed=hd + H + page, scale_key=sk)
    starts, ctxs = _starts_ctx(seqs)
    out = torch.empty_like(qrows).to(DEV)
    K().attn_prefill_mma(qrows.to(DEV), out, kc.to(DEV), vc.to(DEV), bt.to(DEV), starts, ctxs, len(seqs),
                         max(n for _, n in seqs), H, KV, hd, 1.0 / math.sqrt(hd), window)
    r = 0
    for s, (c, n) in enumerate(seqs):
        want = plain.causal_attention(qs[s].double(), ks[s].double(), vs[s].double(), H, KV, hd, window=window or None)[c:]
        assert rel(out[r:r + n], want) <= 2 ** -6, (s, c, n)     # P is rounded to bfloat16 before P V: one more 2^-9 rounding per key
        r += n


@pytest.mark.parametrize("H,KV,hd,page", [(8, 2, 64, 16), (3, 3, 64, 8), (16, 2, 64, 32), (32, 8, 64, 64), (2, 1, 64, 128),
                                          (6, 2, 64, 16), (5, 1, 64, 8), (4, 2, 128, 16), (24, 8, 128, 32), (8, 8, 128, 128), (7, 1, 128, 8)])
def test_attn_prefill_sm100(H, KV, hd, page):
    """The tcgen05 kernel for prompt portions: portions that start mid-page, at a page edge, at
    zero; single tokens beside them; more than one row tile and more than one key tile; one key far
    back scaled so that a wrong or missing key shows. Cache slots no request wrote hold NaN."""
    dt = torch.bfloat16
    seqs = [(5, 6), (0, 3), (2 * page, page), (137, 1), (0, 1), (3 * page - 1, 2), (0, 150), (201, 77), (0, 300), (250, 130)]
    qrows, kc, vc, bt, row_seq, pos, qs, ks, vs = _paged_case(dt, H, KV, hd, page, seqs, seed=hd + H + page,
                                                              scale_key=lambda L: min(3, L - 1), poison=True)
    starts, ctxs = _starts_ctx(seqs)
    out = torch.full_like(qrows, 7.0).to(DEV)
    k = K()
    assert k.attn_prefill_sm100_supported(H, KV, hd, page, bt.shape[1])
    args = (qrows.to(DEV), out, kc.to(DEV), vc.to(DEV), bt.to(DEV), starts, ctxs, len(seqs), max(n for _, n in seqs),
            H, KV, hd, 1.0 / math.sqrt(hd))
    k.attn_prefill_sm100(*args)
    torch.cuda.synchronize()
    k.gemm_sm100_check()
    r = 0
    for s, (c, n) in enumerate(seqs):
        want = plain.causal_attention(qs[s].double(), ks[s].double(), vs[s].double(), H, KV, hd)[c:]
        assert rel(out[r:r + n], want) <= 2 ** -6, (s, c, n)     # P is rounded to bfloat16 before P V
        r += n
    first = out.clone()
    out.fill_(3.0)
    k.attn_prefill_sm100(*args)                                   # nothing needs resetting between launches
    assert torch.equal(out, first)


def test_attn_prefill_sm100_far_key_and_refusals():
    from vllm_oxide_b200.errors import ShapeError
    k = K()
    H, KV, hd, page = 4, 1, 64, 16
    seqs = [(0, 1000), (900, 100)]
    qrows, kc, vc, bt, row_seq, pos, qs, ks, vs = _paged_case(torch.bfloat16, H, KV, hd, page, seqs, seed=5,
                                                              scale_key=lambda L: 3, poison=True)
    starts, ctxs = _starts_ctx(seqs)
    out = torch.empty_like(qrows).to(DEV)
    k.attn_prefill_sm100(qrows.to(DEV), out, kc.to(DEV), vc.to(DEV), bt.to(DEV), starts, ctxs, 2, 1000, H, KV, hd, 0.125)
    r = 0
    for s, (c, n) in enumerate(seqs):
        want = plain.causal_attention(qs[s].double(), ks[s].double(), vs[s].double(), H, KV, hd)[c:]
        assert rel(out[r:r + n], want) <= 2 ** -6, (s, c, n)
        r += n
    k.gemm_sm100_check()
    assert k.attn_prefill_sm100_supported(6, 2, 64, 16, 64) and k.attn_prefill_sm100_supported(4, 2, 128, 16, 64)
    assert not k.attn_prefill_sm100_supported(4, 2, 48, 16, 64) and not k.attn_prefill_sm100_supported(4, 2, 64, 24, 64)
    assert not k.attn_prefill_sm100_supported(4, 2, 64, 4, 64) and not k.attn_prefill_sm100_supported(258, 2, 64, 16, 64)
    assert not k.attn_prefill_sm100_supported(4, 2, 64, 16, 1 << 20)  # the page list would not fit shared memory
    q = torch.zeros(1, 4 * 48, dtype=torch.bfloat16, device=DEV)
    kc6 = torch.zeros(2, 2, 16, 48, dtype=torch.bfloat16, device=DEV)
    z = torch.zeros(2, dtype=torch.int32, device=DEV)
    with pytest.raises(ShapeError, match="not supported"):
        k.attn_prefill_sm100(q, q.clone(), kc6, kc6, torch.zeros(1, 2, dtype=torch.int32, device=DEV), z, z, 1, 1, 4, 2, 48, 1.0)


@pytest.mark.parametrize("splits", [1, 3, 8])
@pytest.mark.parametrize("window", [0, 70])
@pytest.mark.parametrize("H,KV,hd,page", [(8, 2, 64, 16), (3, 1, 64, 8), (4, 4, 128, 32), (32, 2, 128, 16)])
def test_attn_decode_mma(H, KV, hd, page, window, splits):
    dt = torch.bfloat16
    seqs = [(700, 1), (0, 1), (63, 1), (64, 1), (65, 1), (333, 1), (5, 1)]
    sk = (lambda L: max(L - 1 - window, 0)) if window else (lambda L: min(3, L - 1))
    qrows, kc, vc, bt, row_seq, pos, qs, ks, vs = _paged_case(dt, H, KV, hd, page, seqs, seed=hd + H + page + splits, scale_key=sk)
    # a padding row: position -1, attends to nothing, must come out as zeros
    qrows = torch.cat([qrows, torch.randn(1, H * hd).to(dt)])
    pos = torch.cat([pos, torch.tensor([-1], dtype=torch.int32)])
    bt = torch.cat([bt, bt[:1]])
    out = torch.full_like(qrows, 7.0).to(DEV)
    k = K()
    k.attn_decode_mma(qrows.to(DEV), out, kc.to(DEV), vc.to(DEV), bt.to(DEV), pos.to(DEV), H, KV, hd,
                      1.0 / math.sqrt(hd), window, splits)
    for s, (c, n) in enumerate(seqs):
        want = plain.causal_attention(qs[s].double(), ks[s].double(), vs[s].double(), H, KV, hd, window=window or None)[c:]
        assert rel(out[s:s + 1], want) <= 2 ** -6, (s, c)
    assert float(out[len(seqs)].float().abs().max()) == 0.0


@pytest.mark.parametrize("H,KV,hd,page,window,splits", [(8, 2, 64, 16, 0, 37), (6, 2, 128, 32, 0, 64), (4, 4, 64, 8, 300, 19),
                                                        (8, 2, 64, 64, 0, 9)])
def test_attn_decode_mma_merge_through_global_memory(H, KV, hd, page, window, splits):
    """Up to 64 blocks per request without a cluster: long and short requests in one launch (a
    short one uses one block and the others leave), a far key that decides the result, a padding
    row; and a second launch on the same counters, which the first must have left at zero."""
    dt = torch.bfloat16
    seqs = [(5000, 1), (0, 1), (130, 1), (700, 1), (64 * splits * 2 - 1, 1)]
    sk = (lambda L: max(L - 1 - window, 0)) if window else (lambda L: min(3, L - 1))
    qrows, kc, vc, bt, row_seq, pos, qs, ks, vs = _paged_case(dt, H, KV, hd, page, seqs, seed=hd + H + page + splits, scale_key=sk)
    qrows = torch.cat([qrows, torch.randn(1, H * hd).to(dt)])
    pos = torch.cat([pos, torch.tensor([-1], dtype=torch.int32)])
    bt = torch.cat([bt, bt[:1]])
    k = K()
    S = qrows.shape[0]
    partials = torch.full((k.attn_decode_partial_floats(S, KV, hd, splits),), float("nan"), device=DEV)
    arrived = torch.zeros(S * KV, dtype=torch.int32, device=DEV)
    args = (kc.to(DEV), vc.to(DEV), bt.to(DEV), pos.to(DEV), H, KV, hd, 1.0 / math.sqrt(hd), window, splits, partials, arrived)
    for _ in range(2):
        out = torch.full_like(qrows, 7.0).to(DEV)
        k.attn_decode_mma(qrows.to(DEV), out, *args)
        for s, (c, n) in enumerate(seqs):
            want = plain.causal_attention(qs[s].double(), ks[s].double(), vs[s].double(), H, KV, hd, window=window or None)[c:]
            assert rel(out[s:s + 1], want) <= 2 ** -6, (s, c)
        assert float(out[len(seqs)].float().abs().max()) == 0.0
        assert int(arrived.abs().max()) == 0
    from vllm_oxide_b200.errors import ShapeError
    with pytest.raises(ShapeError, match="splits must be"):
        k.attn_decode_mma(qrows.to(DEV), out, *args[:9], 65, partials, arrived)
    with pytest.raises(ShapeError, match="splits must be"):
        k.attn_decode_mma(qrows.to(DEV), out, *args[:9], 9)
    with pytest.raises(ShapeError, match="partials must be"):
        k.attn_decode_mma(qrows.to(DEV), out, *args[:10], partials[:100], arrived)


def test_attn_mma_refusals():
    from vllm_oxide_b200.errors import ShapeError
    k = K()
    assert k.attn_mma_supported(32, 8, 64, 16, True) and k.attn_mma_supported(24, 8, 128, 16, False)
    assert not k.attn_mma_supported(4, 2, 48, 16, False) and not k.attn_mma_supported(4, 2, 64, 24, False)
    assert not k.attn_mma_supported(34, 2, 64, 16, True) and k.attn_mma_supported(34, 2, 64, 16, False)
    q = torch.zeros(1, 4 * 48, dtype=torch.bfloat16, device=DEV)
    kc = torch.zeros(2, 2, 16, 48, dtype=torch.bfloat16, device=DEV)
    z = torch.zeros(2, dtype=torch.int32, device=DEV)
    with pytest.raises(ShapeError, match="not supported"):
        k.attn_prefill_mma(q, q.clone(), kc, kc, torch.zeros(1, 2, dtype=torch.int32, device=DEV), z, z, 1, 1, 4, 2, 48, 1.0)
    with pytest.raises(ShapeError, match="bfloat16 only"):
        k.attn_prefill_mma(q.float(), q.float(), kc.float(), kc.float(), torch.zeros(1, 2, dtype=torch.int32, device=DEV), z, z, 1, 1, 4, 2, 48, 1.0)


# ----------------------------------------------------------------------------- tcgen05 matrix product (bfloat16)
@pytest.mark.parametrize("odt", [torch.bfloat16, torch.float32], ids=["bf16out", "f32out"])
@pytest.mark.parametrize("T,N,Kd,splits", [
    (1, 128, 64, 1), (8, 128, 256, None), (5, 640, 8192, 8), (8, 2048, 2048, 3), (16, 256, 512, 2), (17, 200, 136, None),
    (33, 200, 136, None), (64, 2048, 2048, None), (100, 300, 520, None), (129, 1000, 1032, None), (300, 520, 264, None),
    (700, 384, 96, None)])
def test_gemm_sm100(T, N, Kd, splits, odt):
    """TMA + tcgen05 product against float64: rows and features that are no multiple of a tile,
    K that is no multiple of 64, every token-tile width (16 ... 256), K split over a cluster."""
    g = torch.Generator().manual_seed(T * 7 + N)
    a = torch.randn(T, Kd, generator=g).to(torch.bfloat16).to(DEV)
    w = torch.randn(N, Kd, generator=g).to(torch.bfloat16).to(DEV)
    out = torch.full((T, N), 7.0, dtype=odt, device=DEV)
    k = K()
    k.gemm_sm100(a, w, out, splits)
    torch.cuda.synchronize()
    k.gemm_sm100_check()
    want = plain.linear(a.double().cpu(), w.double().cpu())
    # bfloat16 inputs are exact and products accumulate in float32: sqrt(K) * 2^-24 like the float32
    # kernel; a bfloat16 result adds one rounding of 2^-9
    tol = (2.0 ** -8) if odt == torch.bfloat16 else max(2e-6, 2.0 ** -22 * math.sqrt(Kd))
    assert rel(out, want) <= tol
    # a row's value does not depend on the rows beside it (same tile width): bitwise
    if T > 1:
        bt = 16 if T <= 16 else 32 if T <= 32 else 64 if T <= 64 else 128 if T <= 128 else 256
        lo = max(0, T - 2) if (T - 1) // bt == 0 or bt == 16 else T - 1
        sub = torch.empty((T - lo, N), dtype=odt, device=DEV)
        if (T - lo <= 16) == (T <= 16) and splits == 1:
            k.gemm_sm100(a[lo:].contiguous(), w, sub, splits)
            assert torch.equal(sub, out[lo:])
    # replay: nothing needs resetting between launches
    out2 = torch.zeros_like(out)
    k.gemm_sm100(a, w, out2, splits)
    assert torch.equal(out2, out)


def test_gemm_sm100_strided_and_refusals():
    from vllm_oxide_b200.errors import ShapeError
    k = K()
    g = torch.Generator().manual_seed(1)
    wide = torch.randn(9, 96, generator=g).to(torch.bfloat16).to(DEV)
    w = torch.randn(50, 64, generator=g).to(torch.bfloat16).to(DEV)
    outw = torch.zeros(9, 80, dtype=torch.bfloat16, device=DEV)
    k.gemm_sm100(wide[:, 16:80], w, outw[:, 8:58])             # column slices of wider buffers
    want = plain.linear(wide[:, 16:80].double().cpu(), w.double().cpu())
    assert rel(outw[:, 8:58], want) <= 2 ** -8
    assert float(outw[:, :8].float().abs().max()) == 0.0 and float(outw[:, 58:].float().abs().max()) == 0.0
    assert not k.gemm_sm100_supported(wide[:, 1:65], w)         # rows not 16-byte aligned
    assert not k.gemm_sm100_supported(wide[:, :60], w[:, :60])  # K no multiple of 8
    with pytest.raises(ShapeError):
        k.gemm_sm100(wide[:, :60], w[:, :60], outw[:, :50])
    # linear() falls back to the library product for such operands instead of failing
    o = torch.empty(9, 50, dtype=torch.bfloat16, device=DEV)
    k.linear(wide[:, :60].contiguous(), w[:, :60].contiguous(), o)
    assert rel(o, plain.linear(wide[:, :60].double().cpu(), w[:, :60].double().cpu())) <= 2 ** -8


# ----------------------------------------------------------------------------- fused epilogues of the tcgen05 product
@pytest.mark.parametrize("T,I,Kd,splits", [(1, 128, 64, 1), (8, 8192, 2048, None), (5, 224, 96, 1), (16, 300, 520, 3), (32, 1000, 256, 2), (17, 128, 1024, 8),
                                            (33, 224, 96, 1), (64, 8192, 2048, None), (50, 300, 520, 3)])
def test_gemm_swiglu(T, I, Kd, splits):
    g = torch.Generator().manual_seed(T + I)
    a = torch.randn(T, Kd, generator=g).to(torch.bfloat16).to(DEV)
    w = (torch.randn(2 * I, Kd, generator=g) / math.sqrt(Kd) * 2).to(torch.bfloat16).to(DEV)
    out = torch.full((T, I), 7.0, dtype=torch.bfloat16, device=DEV)
    k = K()
    k.gemm_swiglu(a, w, out, splits)
    torch.cuda.synchronize()
    k.gemm_sm100_check()
    gate = plain.linear(a.double().cpu(), w[:I].double().cpu())
    up = plain.linear(a.double().cpu(), w[I:].double().cpu())
    assert rel(out, plain.swiglu(gate, up)) <= 2 ** -8
    out2 = torch.zeros_like(out)
    k.gemm_swiglu(a, w, out2, splits)
    assert torch.equal(out, out2)


@pytest.mark.parametrize("rope", [True, False])
@pytest.mark.parametrize("T,H,KV,hd,Kd,page,splits", [(8, 32, 8, 64, 2048, 16, None), (1, 4, 2, 64, 128, 16, 1), (13, 3, 1, 32, 96, 8, 1),
                                                      (32, 6, 2, 16, 200, 8, 2), (5, 2, 2, 128, 512, 32, 4), (20, 5, 5, 64, 320, 16, 5),
                                                      (64, 32, 8, 64, 2048, 16, None), (41, 3, 1, 32, 96, 8, 2)])
def test_gemm_qkv_rope(T, H, KV, hd, Kd, page, splits, rope):
    g = torch.Generator().manual_seed(T + H + hd)
    a = torch.randn(T, Kd, generator=g).to(torch.bfloat16).to(DEV)
    w = (torch.randn((H + 2 * KV) * hd, Kd, generator=g) / math.sqrt(Kd)).to(torch.bfloat16).to(DEV)
    cfg = {"head_dim": hd, "hidden_size": H * hd, "num_attention_heads": H, "rope_theta": 500000.0,
           "rope_scaling": {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                            "original_max_position_embeddings": 64}}
    inv = plain.rope_inv_freq(cfg)
    positions = [(37 * i + 5) % 3000 for i in range(T)]
    pages = -(-T // page) + 4
    slots = torch.randperm(pages * page, generator=g)[:T].to(torch.int32)
    if T > 2:
        slots[2] = -1                                                   # this token writes nothing
    kc = torch.full((pages, KV, page, hd), 7.0, dtype=torch.bfloat16, device=DEV)
    vc = torch.full((pages, KV, page, hd), 7.0, dtype=torch.bfloat16, device=DEV)
    q = torch.full((T, H * hd), 7.0, dtype=torch.bfloat16, device=DEV)
    k = K()
    k.gemm_qkv_rope(a, w, q, torch.tensor(positions, dtype=torch.int32, device=DEV), slots.to(DEV),
                    inv.to(DEV) if rope else None, kc, vc, H, KV, hd, splits)
    torch.cuda.synchronize()
    k.gemm_sm100_check()
    qkv = plain.linear(a.double().cpu(), w.double().cpu())
    wq, wk, wv = qkv[:, :H * hd], qkv[:, H * hd:(H + KV) * hd], qkv[:, (H + KV) * hd:]
    if rope:
        wq, wk = plain.rope(wq, positions, inv, hd), plain.rope(wk, positions, inv, hd)
    assert rel(q, wq) <= 2 ** -8
    written = set()
    for t in range(T):
        s_ = int(slots[t])
        if s_ < 0:
            continue
        written.add(s_)
        pg, off = s_ // page, s_ % page
        assert rel(kc[pg, :, off, :].reshape(-1), wk[t]) <= 2 ** -8
        assert rel(vc[pg, :, off, :].reshape(-1), wv[t]) <= 2 ** -8
    for s_ in range(pages * page):
        if s_ not in written:
            assert float((kc[s_ // page, :, s_ % page, :].float() - 7.0).abs().max()) == 0.0
            assert float((vc[s_ // page, :, s_ % page, :].float() - 7.0).abs().max()) == 0.0


def test_fused_gemm_refusals():
    from vllm_oxide_b200.errors import ShapeError
    k = K()
    a = torch.zeros(70, 64, dtype=torch.bfloat16, device=DEV)
    w = torch.zeros(256, 64, dtype=torch.bfloat16, device=DEV)
    with pytest.raises(ShapeError, match="at most 64"):
        k.gemm_swiglu(a, w, torch.zeros(70, 128, dtype=torch.bfloat16, device=DEV))
    assert not k.gemm_qkv_rope_supported(48) and k.gemm_qkv_rope_supported(64)


def _folded_input(T, Kd, g):
    """A residual x [T, Kd], the next norm's weight, and what the folded form hands to a product:
    bf16(x * weight) and the sums of squares of x per 128-feature tile."""
    x = torch.randn(T, Kd, generator=g) * 1.5
    wn = 1.0 + 0.3 * torch.randn(Kd, generator=g)
    xn = (x * wn).to(torch.bfloat16)
    tiles = -(-Kd // 128)
    ssq = torch.zeros(tiles, 64)
    for i in range(tiles):
        ssq[i, :T] = (x[:, i * 128:(i + 1) * 128] ** 2).sum(1)
    return x, wn, xn, ssq


@pytest.mark.parametrize("T,N,Kd,splits", [(1, 128, 128, 1), (8, 2048, 2048, None), (20, 200, 320, 2), (32, 640, 8192, 8),
                                           (33, 200, 320, 1), (64, 2048, 8192, None), (47, 384, 256, 3)])
def test_gemm_fused_residual_and_folded_norm(T, N, Kd, splits):
    """EPI_RESID with the RMSNorm of the input folded in: resid += rmsnorm(x) W^T (the norm as a
    per-token scale of the accumulator), the next norm's input bf16(resid * next_w) and the
    per-tile sums of squares of the new residual come out of the same kernel."""
    from vllm_oxide_b200.kernels import EPI_RESID, EPI_STORE
    g = torch.Generator().manual_seed(T * 3 + N)
    eps = 1e-5
    x, wn, xn, ssq = _folded_input(T, Kd, g)
    w = (torch.randn(N, Kd, generator=g) / math.sqrt(Kd)).to(torch.bfloat16)
    resid0 = torch.randn(T, N, generator=g)
    next_w = 1.0 + 0.3 * torch.randn(N, generator=g)
    k = K()
    resid = resid0.clone().to(DEV)
    xn_out = torch.full((T, N), 7.0, dtype=torch.bfloat16, device=DEV)
    ssq_out = torch.full((-(-N // 128), 64), 7.0, device=DEV)
    k.gemm_fused(xn.to(DEV), w.to(DEV), None, EPI_RESID, N, ssq_in=ssq.to(DEV), eps=eps,
                 resid=(resid, next_w.to(DEV), xn_out, ssq_out), splits=splits)
    torch.cuda.synchronize()
    k.gemm_sm100_check()
    # the plain norm of x with weight wn (x * wn rounded to bfloat16 as the kernel's operand), then the product
    inv = 1.0 / torch.sqrt((x.double() ** 2).mean(1) + eps)
    want_delta = plain.linear(xn.double(), w.double()) * inv[:, None]
    want_resid = resid0.double() + want_delta
    assert rel(resid, want_resid) <= max(2e-6, 2.0 ** -22 * math.sqrt(Kd)) * 4
    assert rel(xn_out, want_resid * next_w.double()) <= 2 ** -8
    got = resid.double().cpu()
    for i in range(-(-N // 128)):
        want_ssq = (got[:, i * 128:(i + 1) * 128] ** 2).sum(1)
        assert rel(ssq_out[i, :T], want_ssq) <= 1e-5
    # the same scale on a plain store
    out = torch.empty(T, N, device=DEV)
    k.gemm_fused(xn.to(DEV), w.to(DEV), out, EPI_STORE, N, ssq_in=ssq.to(DEV), eps=eps, splits=splits)
    assert rel(out, want_delta) <= max(2e-6, 2.0 ** -22 * math.sqrt(Kd)) * 4


# ----------------------------------------------------------------------------- tcgen05 product on pairs of SMs
@pytest.mark.parametrize("odt", [torch.bfloat16, torch.float32], ids=["bf16out", "f32out"])
@pytest.mark.parametrize("T,N,Kd", [(1, 8, 64), (256, 256, 64), (300, 520, 264), (129, 1000, 1032), (700, 384, 96), (1030, 2048, 512)])
def test_gemm_sm100_pair(T, N, Kd, odt):
    """The two-SM product (tcgen05.mma.cta_group::2) against float64: rows and features that are no
    multiple of a tile, K that is no multiple of 64, one tile and many, both output types."""
    g = torch.Generator().manual_seed(T * 5 + N)
    a = torch.randn(T, Kd, generator=g).to(torch.bfloat16).to(DEV)
    w = torch.randn(N, Kd, generator=g).to(torch.bfloat16).to(DEV)
    out = torch.full((T, N), 7.0, dtype=odt, device=DEV)
    k = K()
    k.gemm_sm100_pair(a, w, out)
    torch.cuda.synchronize()
    k.gemm_sm100_check()
    want = plain.linear(a.double().cpu(), w.double().cpu())
    tol = (2.0 ** -8) if odt == torch.bfloat16 else max(2e-6, 2.0 ** -22 * math.sqrt(Kd))
    assert rel(out, want) <= tol
    out2 = torch.zeros_like(out)
    k.gemm_sm100_pair(a, w, out2)                                # nothing needs resetting between launches
    assert torch.equal(out2, out)
    # a row's value does not depend on the rows beside it
    if T > 2:
        sub = torch.empty((2, N), dtype=odt, device=DEV)
        k.gemm_sm100_pair(a[T - 2:].contiguous(), w, sub)
        assert torch.equal(sub, out[T - 2:])


def test_gemm_sm100_pair_narrow_output_rows():
    """An output whose rows are not 16-byte aligned takes the element-wise store path."""
    g = torch.Generator().manual_seed(3)
    a = torch.randn(200, 128, generator=g).to(torch.bfloat16).to(DEV)
    w = torch.randn(100, 128, generator=g).to(torch.bfloat16).to(DEV)
    wide = torch.full((200, 101), 7.0, dtype=torch.bfloat16, device=DEV)
    k = K()
    k.gemm_sm100_pair(a, w, wide[:, :100])
    assert rel(wide[:, :100], plain.linear(a.double().cpu(), w.double().cpu())) <= 2 ** -8
    assert float((wide[:, 100].float() - 7.0).abs().max()) == 0.0


@pytest.mark.parametrize("T,I,Kd", [(1, 64, 64), (256, 128, 64), (300, 300, 264), (700, 224, 96), (1100, 1000, 256)])
def test_gemm_pair_swiglu(T, I, Kd):
    g = torch.Generator().manual_seed(T + I)
    a = torch.randn(T, Kd, generator=g).to(torch.bfloat16).to(DEV)
    w = (torch.randn(2 * I, Kd, generator=g) / math.sqrt(Kd) * 2).to(torch.bfloat16).to(DEV)
    out = torch.full((T, I), 7.0, dtype=torch.bfloat16, device=DEV)
    k = K()
    k.gemm_pair_swiglu(a, w, out)
    torch.cuda.synchronize()
    k.gemm_sm100_check()
    gate = plain.linear(a.double().cpu(), w[:I].double().cpu())
    up = plain.linear(a.double().cpu(), w[I:].double().cpu())
    assert rel(out, plain.swiglu(gate, up)) <= 2 ** -8
    out2 = torch.zeros_like(out)
    k.gemm_pair_swiglu(a, w, out2)
    assert torch.equal(out, out2)


def test_a_wait_that_runs_out_raises_the_error_word_and_harms_nothing():
    """The give-up path of the tensor-core kernels: a one-block launch of the few-token product is
    told to expect 16 bytes more than its loads bring, with the wait limit lowered to 10 ms. The
    kernel returns (no hang, no fault), the error word turns into a KernelError, and the next
    ordinary launch on the same context is correct."""
    from vllm_oxide_b200 import kernels
    from vllm_oxide_b200.errors import KernelError
    g = torch.Generator().manual_seed(90)
    a = torch.randn(8, 256, generator=g).to(torch.bfloat16).to(DEV)
    w = torch.randn(128, 256, generator=g).to(torch.bfloat16).to(DEV)
    out = torch.zeros(8, 128, dtype=torch.float32, device=DEV)
    kernels.gemm_sm100(a, w, out, splits=1)
    torch.cuda.synchronize()
    kernels.gemm_sm100_check()                                   # nothing wrong so far
    want = a.double().cpu() @ w.double().cpu().t()
    assert rel(out.cpu(), want) <= 1e-5
    kernels.gemm_sm100_test_hooks(extra_tx_bytes=16, wait_limit_ms=10.0)
    try:
        kernels.gemm_sm100(a, w, torch.zeros_like(out), splits=1)
        torch.cuda.synchronize()                           # returns after some 10 ms
    finally:
        kernels.gemm_sm100_test_hooks(0, 0.0)
    with pytest.raises(KernelError, match="bounded wait"):
        kernels.gemm_sm100_check()
    kernels.gemm_sm100_check()                                   # the word was cleared by the check
    out2 = torch.zeros_like(out)
    kernels.gemm_sm100(a, w, out2, splits=1)
    big = torch.zeros(8, 2048, dtype=torch.float32, device=DEV)
    w2 = torch.randn(2048, 256, generator=g).to(torch.bfloat16).to(DEV)
    kernels.gemm_sm100(a, w2, big)                               # and a launch with a cluster split
    torch.cuda.synchronize()
    kernels.gemm_sm100_check()
    assert rel(out2.cpu(), want) <= 1e-5
    assert rel(big.cpu(), a.double().cpu() @ w2.double().cpu().t()) <= 1e-5


@pytest.mark.parametrize("T,V,Kd", [(1, 128, 64), (8, 128256, 256), (5, 1000, 96), (16, 301, 128), (33, 5000, 64), (64, 2048, 320)])
def test_output_head_that_picks_in_its_epilogue(T, V, Kd):
    """EPI_PICK + pick_final against the logits (EPI_STORE) + pick_tokens: the same tokens for greedy
    and sampled rows, ties kept at the first index, a NaN row flagged, with the folded norm's scale."""
    from vllm_oxide_b200 import kernels
    g = torch.Generator().manual_seed(V + T)
    x, wn, xn, ssq = _folded_input(T, Kd, g)
    w = (torch.randn(V, Kd, generator=g) * 0.2).to(torch.bfloat16)
    if V > 40:
        w[37] = w[11]                                      # a tie between two logits of every row: the first index wins
        w[V - 1] = w[11]
    w, xn, ssq = w.to(DEV), xn.to(DEV), ssq.to(DEV)
    if T > 2:
        xn[2] = float("nan")                               # row 2 holds NaN logits
    temps = torch.tensor([0.0 if i % 3 else 0.8 for i in range(T)], device=DEV)
    temps[0] = 0.0
    seeds = torch.tensor([[i + 1, 7 * i] for i in range(T)], dtype=torch.int32, device=DEV)
    steps = torch.arange(T, dtype=torch.int32, device=DEV) + 3
    logits = torch.empty(T, V, dtype=torch.float32, device=DEV)
    kernels.gemm_fused(xn, w, logits, kernels.EPI_STORE, V, ssq_in=ssq, eps=1e-5)
    sp = kernels.pick_splits(V)
    want = torch.zeros(T, dtype=torch.int32, device=DEV)
    kernels.pick_tokens(logits, want, torch.zeros(T, dtype=torch.int32, device=DEV), torch.empty(T * sp, device=DEV),
                        torch.empty(T * sp, dtype=torch.int32, device=DEV), temps, seeds, steps)
    tiles = kernels.pick_tiles(V)
    pv = torch.full((T, tiles + 3), float("nan"), device=DEV)
    pi = torch.full((T, tiles + 3), -5, dtype=torch.int32, device=DEV)
    flags = torch.zeros(T, dtype=torch.int32, device=DEV)
    got = torch.full((T,), -9, dtype=torch.int32, device=DEV)
    kernels.gemm_fused(xn, w, None, kernels.EPI_PICK, V, ssq_in=ssq, eps=1e-5, pick=(temps, seeds, steps, pv, pi, flags))
    kernels.pick_final(pv[:, :tiles].contiguous(), pi[:, :tiles].contiguous(), T, V, flags, got)
    assert got.tolist() == want.tolist()
    if T > 2:
        assert got[2].item() == -1 and int(flags.sum()) == 0          # flagged, and the flag was put back
    if V > 40:
        assert got[0].item() != 37 and got[0].item() != V - 1         # never the later twin of a tie
    # greedy without sampling parameters at all
    got2 = torch.full((T,), -9, dtype=torch.int32, device=DEV)
    kernels.gemm_fused(xn, w, None, kernels.EPI_PICK, V, ssq_in=ssq, eps=1e-5, pick=(None, None, None, pv, pi, flags))
    kernels.pick_final(pv[:, :tiles].contiguous(), pi[:, :tiles].contiguous(), T, V, flags, got2)
    ref = torch.where(torch.isnan(logits).any(1), torch.full_like(want, -1), logits.argmax(1).to(torch.int32))
    assert got2.tolist() == ref.tolist()
