"""Each kernel alone against a plain reference of the same operation, at sizes other
than the engine's test models."""
import math

import numpy as np
import pytest
import torch

import plain_qwen3 as plain

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _ops():
    from skyla_kernel_b200.kernels import ops
    return ops


def _rand(*shape, seed=0, dtype=torch.float32, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(*shape, generator=g) * scale).to(dtype).to(DEV)


def _tol(dtype):
    return dict(rtol=2e-2, atol=2e-2) if dtype == torch.bfloat16 else dict(rtol=1e-5, atol=1e-5)


@pytest.mark.parametrize("width", [48, 80, 1000, 4096])
@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16])
def test_rmsnorm(width, out_dtype):
    ops = _ops()
    x = _rand(9, width, seed=1, scale=3.0)
    w = 1 + 0.1 * _rand(width, seed=2)
    out = torch.empty(9, width, dtype=out_dtype, device=DEV)
    ops.rmsnorm(x, w, 1e-5, out)
    ref = plain.rmsnorm(x.cpu(), w.cpu(), 1e-5)
    torch.testing.assert_close(out.float().cpu(), ref, **_tol(out_dtype))
    rows = torch.tensor([8, 0, 3], dtype=torch.int32, device=DEV)
    out2 = torch.empty(3, width, dtype=out_dtype, device=DEV)
    ops.rmsnorm(x, w, 1e-5, out2, rows)
    assert torch.equal(out2, out[rows.long()])  # the same row gives the same bits wherever it lies


def test_embed_gather():
    ops = _ops()
    for dt in (torch.float32, torch.bfloat16):
        table = _rand(131, 80, seed=3, dtype=dt)
        toks = torch.tensor([130, 0, 5, 5, 77], dtype=torch.int32, device=DEV)
        out = torch.empty(5, 80, dtype=torch.float32, device=DEV)
        ops.embed_gather(toks, table, out)
        assert torch.equal(out, table[toks.long()].float())


@pytest.mark.parametrize("m,n,k", [(1, 131, 80), (5, 64, 64), (70, 96, 160), (130, 509, 96)])
@pytest.mark.parametrize("xdt,wdt", [(torch.float32, torch.float32), (torch.bfloat16, torch.bfloat16),
                                      (torch.bfloat16, torch.float32)])
def test_linear_plain_store_and_accumulate(m, n, k, xdt, wdt):
    ops = _ops()
    x, w = _rand(m, k, seed=4, dtype=xdt), _rand(n, k, seed=5, dtype=wdt, scale=0.1)
    ref = (x.double() @ w.double().T).float()
    y = torch.empty(m, n, dtype=xdt, device=DEV)
    ops.linear_plain(x, w, y, ops.STORE)
    torch.testing.assert_close(y.float(), ref, **_tol(xdt))
    acc = _rand(m, n, seed=6)
    before = acc.clone()
    ops.linear_plain(x, w, acc, ops.ACCUMULATE)
    torch.testing.assert_close(acc, before + ref, rtol=1e-4, atol=1e-4)
    # a row's result does not depend on the rows around it
    r = min(3, m - 1)
    y1 = torch.empty(1, n, dtype=xdt, device=DEV)
    ops.linear_plain(x[r:r + 1], w, y1, ops.STORE)
    assert torch.equal(y1[0], y[r])


@pytest.mark.parametrize("group", [None, 16])
@pytest.mark.parametrize("dt", [torch.float32, torch.bfloat16])
def test_linear_plain_gated(group, dt):
    ops = _ops()
    m, n, k = 37, 112, 80
    x, g, u = _rand(m, k, seed=7, dtype=dt), _rand(n, k, seed=8, dtype=dt, scale=0.2), _rand(n, k, seed=9, dtype=dt, scale=0.2)
    grp = group or n
    w = torch.stack((g.reshape(n // grp, grp, k), u.reshape(n // grp, grp, k)), dim=1).reshape(2 * n, k).contiguous()
    y = torch.empty(m, n, dtype=dt, device=DEV)
    ops.linear_plain(x, w, y, ops.GATED, grp)
    ref = plain.silu(x.double().cpu() @ g.double().cpu().T) * (x.double().cpu() @ u.double().cpu().T)
    torch.testing.assert_close(y.float().cpu(), ref.float(), **_tol(dt))


def _paged(n_seqs, lens, nkv, hd, dtype, seed, page_size=64, shuffle=True):
    """Random keys/values per sequence scattered over shuffled pages; returns pools, table, dense copies."""
    g = torch.Generator().manual_seed(seed)
    P = max(-(-l // page_size) for l in lens)
    n_pages = n_seqs * P + 3
    order = torch.randperm(n_pages, generator=g).tolist() if shuffle else list(range(n_pages))
    table = torch.zeros(n_seqs, P, dtype=torch.int32)
    k_pool = torch.zeros(n_pages, nkv, page_size, hd, dtype=dtype)
    v_pool = torch.zeros(n_pages, nkv, page_size, hd, dtype=dtype)
    ks, vs = [], []
    for b, l in enumerate(lens):
        k = torch.randn(l, nkv, hd, generator=g).to(dtype)
        v = torch.randn(l, nkv, hd, generator=g).to(dtype)
        ks.append(k); vs.append(v)
        for j in range(-(-l // page_size)):
            pg = order.pop()
            table[b, j] = pg
            seg = slice(j * page_size, min(l, (j + 1) * page_size))
            k_pool[pg, :, : seg.stop - seg.start] = k[seg].transpose(0, 1)
            v_pool[pg, :, : seg.stop - seg.start] = v[seg].transpose(0, 1)
    return k_pool.to(DEV), v_pool.to(DEV), table.to(DEV), ks, vs


def _attn_ref(q, k, v, pos, nq, nkv, scale, window):
    """q [nq, hd] at position pos over k, v [len, nkv, hd] (float64)."""
    out = []
    first = max(0, pos - window + 1) if window else 0
    for h in range(nq):
        kvh = h // (nq // nkv)
        s = (k[first:pos + 1, kvh].double() @ q[h].double()) * scale
        p = torch.softmax(s, 0)
        out.append(p @ v[first:pos + 1, kvh].double())
    return torch.stack(out)


@pytest.mark.parametrize("nq,nkv,hd", [(4, 2, 16), (6, 1, 32), (3, 3, 48), (8, 2, 128), (5, 5, 80)])
@pytest.mark.parametrize("dt", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("window", [0, 70])
def test_attention_plain(nq, nkv, hd, dt, window):
    ops = _ops()
    lens = [1, 64, 65, 200, 333]
    k_pool, v_pool, table, ks, vs = _paged(len(lens), lens, nkv, hd, dt, seed=nq * 100 + hd)
    # tokens: for every sequence its last position, plus some inner ones of the long sequences
    toks = [(b, l - 1) for b, l in enumerate(lens)] + [(3, 63), (3, 64), (4, 128), (4, 5)]
    q = _rand(len(toks), nq * hd, seed=11, dtype=dt)
    out = torch.empty(len(toks), nq * hd, dtype=dt, device=DEV)
    tok_pos = torch.tensor([p for _, p in toks], dtype=torch.int32, device=DEV)
    tok_seq = torch.tensor([b for b, _ in toks], dtype=torch.int32, device=DEV)
    scale = 1.0 / math.sqrt(hd)
    ops.attention_plain(q, out, nq, nkv, hd, k_pool, v_pool, table, 64, tok_pos, tok_seq, scale, window)
    for i, (b, p) in enumerate(toks):
        ref = _attn_ref(q[i].cpu().view(nq, hd), ks[b], vs[b], p, nq, nkv, scale, window)
        torch.testing.assert_close(out[i].float().cpu().view(nq, hd), ref.float(), **_tol(dt))


@pytest.mark.parametrize("dt", [torch.float32, torch.bfloat16])
def test_attention_finds_one_far_key(dt):
    """One key among hundreds is made to stand out; the output must be its value."""
    ops = _ops()
    nq, nkv, hd, L = 4, 2, 32, 700
    k_pool, v_pool, table, ks, vs = _paged(1, [L], nkv, hd, dt, seed=5)
    q = _rand(1, nq * hd, seed=12, dtype=dt)
    for target in (0, 63, 64, 411, L - 1):
        kp = k_pool.clone()
        page, off = int(table[0, target // 64]), target % 64
        for kvh in range(nkv):
            qh = q[0].view(nq, hd)[kvh * 2].float()
            kp[page, kvh, off] = (qh / qh.norm() * 60.0).to(dt)  # score ~ 60*|q|/sqrt(hd) for heads of this group
        out = torch.empty(1, nq * hd, dtype=dt, device=DEV)
        ops.attention_plain(q, out, nq, nkv, hd, kp, v_pool, table, 64, torch.tensor([L - 1], dtype=torch.int32, device=DEV),
                            torch.zeros(1, dtype=torch.int32, device=DEV), 1.0, 0)
        for kvh in range(nkv):
            got = out[0].view(nq, hd)[kvh * 2].float().cpu()
            torch.testing.assert_close(got, vs[0][target, kvh].float(), rtol=2e-2, atol=2e-2)


@pytest.mark.parametrize("nq,nkv,hd,n_rot", [(4, 2, 16, 16), (6, 1, 32, 32), (3, 3, 48, 24), (2, 2, 128, 128)])
@pytest.mark.parametrize("dt", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("use_norm", [True, False])
def test_qk_norm_rope_cache(nq, nkv, hd, n_rot, dt, use_norm):
    ops = _ops()
    T = 7
    positions = [0, 1, 63, 64, 130, 5, 64]
    seqs = [0, 0, 0, 0, 0, 1, 1]
    table = torch.tensor([[4, 2, 6], [1, 5, 0]], dtype=torch.int32, device=DEV)
    width = (nq + 2 * nkv) * hd
    qkv = _rand(T, width, seed=13, dtype=dt)
    orig = qkv.clone()
    qn, kn = 1 + 0.2 * _rand(hd, seed=14), 1 + 0.2 * _rand(hd, seed=15)
    freqs, _ = plain.rope_frequencies(n_rot, 10000.0)
    ang = (torch.arange(200, dtype=torch.float32)[:, None] * freqs[None, :]).double()
    cos, sin = torch.cos(ang).float().to(DEV), torch.sin(ang).float().to(DEV)
    k_pool = torch.zeros(7, nkv, 64, hd, dtype=dt, device=DEV)
    v_pool = torch.zeros_like(k_pool)
    ops.qk_norm_rope_cache(qkv, 0, nq * hd, (nq + nkv) * hd, nq, nkv, hd, qn if use_norm else None,
                           kn if use_norm else None, 1e-6, cos, sin, n_rot,
                           torch.tensor(positions, dtype=torch.int32, device=DEV),
                           torch.tensor(seqs, dtype=torch.int32, device=DEV), k_pool, v_pool, table, 64)
    o = orig.float().cpu()
    pos_t = torch.tensor(positions)
    q = o[:, : nq * hd].view(T, nq, hd)
    k = o[:, nq * hd:(nq + nkv) * hd].view(T, nkv, hd)
    v = o[:, (nq + nkv) * hd:].view(T, nkv, hd)
    if use_norm:
        q, k = plain.rmsnorm(q, qn.cpu(), 1e-6), plain.rmsnorm(k, kn.cpu(), 1e-6)
    q, k = plain.rope_neox(q, pos_t, freqs, 1.0, n_rot), plain.rope_neox(k, pos_t, freqs, 1.0, n_rot)
    tol = _tol(dt)
    torch.testing.assert_close(qkv[:, : nq * hd].float().cpu().view(T, nq, hd), q, **tol)
    assert torch.equal(qkv[:, nq * hd:], orig[:, nq * hd:])  # k and v rows of the buffer are untouched
    for t in range(T):
        page = int(table[seqs[t], positions[t] // 64])
        torch.testing.assert_close(k_pool[page, :, positions[t] % 64].float().cpu(), k[t], **tol)
        torch.testing.assert_close(v_pool[page, :, positions[t] % 64].float().cpu(), v[t], **tol)
    written = {(int(table[seqs[t], positions[t] // 64]), positions[t] % 64) for t in range(T)}
    mask = torch.ones(7, 64, dtype=torch.bool)
    for pg, off in written:
        mask[pg, off] = False
    assert (k_pool.float().cpu().abs().sum((1, 3))[mask] == 0).all()  # nothing else was written


def test_refused_sizes_are_errors_not_wrong_results():
    ops = _ops()
    from skyla_kernel_b200.kernels import KernelError
    with pytest.raises(KernelError, match="head size"):
        ops.attention_plain(_rand(1, 1024), torch.empty(1, 1024, device=DEV), 1, 1, 1024,
                            torch.zeros(1, 1, 64, 1024, device=DEV), torch.zeros(1, 1, 64, 1024, device=DEV),
                            torch.zeros(1, 1, dtype=torch.int32, device=DEV), 64,
                            torch.zeros(1, dtype=torch.int32, device=DEV), torch.zeros(1, dtype=torch.int32, device=DEV), 1.0)
    with pytest.raises(KernelError):
        ops.rmsnorm(torch.zeros(2, 8), torch.ones(8), 1e-5, torch.zeros(2, 8))  # host tensors: no CPU path
    with pytest.raises(KernelError, match="float32 or bfloat16"):
        ops.linear_plain(torch.zeros(2, 8, dtype=torch.float16, device=DEV), torch.zeros(4, 8, dtype=torch.float16, device=DEV),
                         torch.zeros(2, 4, dtype=torch.float16, device=DEV))


def test_greedy_takes_lowest_index_among_equals():
    ops = _ops()
    logits = torch.full((3, 509), -1.0, device=DEV)
    logits[0, [400, 17, 300]] = 2.0
    logits[1, 508] = 5.0
    logits[2, 0] = 0.5
    out = torch.empty(3, dtype=torch.int32, device=DEV)
    ops.sample(logits, out)
    assert out.tolist() == [17, 508, 0]


@pytest.mark.parametrize("temperature,top_k,top_p", [(0.8, 0, 1.0), (1.0, 5, 1.0), (0.6, 40, 0.95), (1.3, 0, 0.7)])
def test_sampling_matches_its_plain_twin(temperature, top_k, top_p):
    ops = _ops()
    V, R = 1031, 24
    logits = _rand(R, V, seed=21, scale=2.5)
    req = torch.arange(R, dtype=torch.int32, device=DEV) % 5
    steps = torch.arange(R, dtype=torch.int32, device=DEV) // 5
    out = torch.empty(R, dtype=torch.int32, device=DEV)
    ops.sample(logits, out, temperature, top_k, top_p, 1234567890123, req, steps)
    for r in range(R):
        scores, keep = plain.sample_scores(logits[r].cpu(), temperature, top_k, top_p, 1234567890123,
                                           int(req[r]), int(steps[r]))
        tok = int(out[r])
        assert keep[tok], f"row {r}: token {tok} is outside the kept set"
        best = np.max(scores)
        assert scores[tok] >= best - 1e-4, f"row {r}: drew {tok} ({scores[tok]}), twin's best is {best}"
    # a row's draw depends on its own keys only, not on its neighbours
    out2 = torch.empty(1, dtype=torch.int32, device=DEV)
    ops.sample(logits[7:8], out2, temperature, top_k, top_p, 1234567890123, req[7:8].contiguous(), steps[7:8].contiguous())
    assert int(out2[0]) == int(out[7])


def test_sampling_frequencies_follow_softmax():
    ops = _ops()
    logits = torch.tensor([[0.0, 3.0, 1.0, 2.9, -1.0, 2.0]], device=DEV).repeat(4000, 1)
    out = torch.empty(4000, dtype=torch.int32, device=DEV)
    ops.sample(logits, out, 1.0, 0, 1.0, 77, torch.zeros(4000, dtype=torch.int32, device=DEV),
               torch.arange(4000, dtype=torch.int32, device=DEV))
    freq = torch.bincount(out.long().cpu(), minlength=6).double() / 4000
    assert (freq - torch.softmax(logits[0].double().cpu(), 0)).abs().max() < 0.03


def test_fill_normal_and_bandwidth_probe():
    ops = _ops()
    for dt in (torch.float32, torch.bfloat16):
        t = torch.empty(1_000_001, dtype=dt, device=DEV)
        ops.fill_normal(t, 1.0, 0.02, 5)
        assert abs(t.float().mean().item() - 1.0) < 1e-3 and abs(t.float().std().item() - 0.02) < 1e-3
        t2 = torch.empty_like(t)
        ops.fill_normal(t2, 1.0, 0.02, 5)
        assert torch.equal(t, t2)
    buf = torch.ones(1 << 22, dtype=torch.int32, device=DEV)
    sink = torch.zeros(1, dtype=torch.int32, device=DEV)
    ops.bandwidth_read(buf, 296, sink)
    torch.cuda.synchronize()
    assert int(sink[0]) == 0


# ------------------------------------------------------------- tensor-core GEMM
@pytest.mark.parametrize("m,n,k", [(1, 131, 80), (8, 256, 64), (16, 128, 4096), (17, 509, 96), (70, 96, 160),
                                   (130, 384, 1032), (300, 200, 264), (1000, 640, 512)])
def test_gemm_tc_store_and_accumulate(m, n, k):
    ops = _ops()
    x = _rand(m, k, seed=31, dtype=torch.bfloat16)
    w = _rand(n, k, seed=32, dtype=torch.bfloat16, scale=0.1)
    ref = (x.double() @ w.double().T)
    scale = ref.abs().max().item()
    wm = ops.TensorMap(w, 128)
    y32 = torch.full((m, n), float("nan"), dtype=torch.float32, device=DEV)
    ops.gemm_tc(x, wm, n, y32, ops.TC_STORE_F32)
    assert (y32.double() - ref).abs().max().item() <= 2e-5 * scale + 1e-6
    y16 = torch.empty(m, n, dtype=torch.bfloat16, device=DEV)
    ops.gemm_tc(x, wm, n, y16, ops.TC_STORE_BF16)
    assert torch.equal(y16, y32.to(torch.bfloat16))
    acc = _rand(m, n, seed=33)
    before = acc.clone()
    ops.gemm_tc(x, wm, n, acc, ops.TC_ACCUM_F32)
    assert (acc.double() - before.double() - ref).abs().max().item() <= 2e-5 * scale + 1e-5
    # every token tile width gives the same numbers for the rows it holds
    for bn in ops.TC_TOKEN_TILES:
        y = torch.empty(m, n, dtype=torch.float32, device=DEV)
        ops.gemm_tc(x, wm, n, y, ops.TC_STORE_F32, bn=bn)
        assert (y.double() - ref).abs().max().item() <= 2e-5 * scale + 1e-6, f"token tile {bn}"
    ops.check_device_errors(DEV)


@pytest.mark.parametrize("m,n,k", [(1, 128, 64), (9, 256, 80), (70, 384, 160), (200, 128, 520), (33, 200, 72),
                                   (300, 1000, 328)])
def test_gemm_tc_gated(m, n, k):
    ops = _ops()
    from skyla_kernel_b200.parts.feedforward import fuse_gate_up
    x = _rand(m, k, seed=36, dtype=torch.bfloat16)
    g, u = _rand(n, k, seed=37, dtype=torch.bfloat16, scale=0.2), _rand(n, k, seed=38, dtype=torch.bfloat16, scale=0.2)
    w = fuse_gate_up(g, u)
    y = torch.empty(m, n, dtype=torch.bfloat16, device=DEV)
    ops.gemm_tc(x, ops.TensorMap(w, 128), n, y, ops.TC_GLU_BF16)
    gd, ud = x.double() @ g.double().T, x.double() @ u.double().T
    ref = gd / (1 + torch.exp(-gd)) * ud
    torch.testing.assert_close(y.double(), ref, rtol=1e-2, atol=1e-2 * ref.abs().max().item())
    plain_y = torch.empty_like(y)
    ops.linear_plain(x, w, plain_y, ops.GATED)  # the plain twin on the same fused matrix
    torch.testing.assert_close(y.float(), plain_y.float(), rtol=2e-2, atol=1e-3)
    ops.check_device_errors(DEV)


def test_gemm_tc_refuses_what_it_cannot_do():
    ops = _ops()
    from skyla_kernel_b200.kernels import KernelError
    x = _rand(4, 100, seed=1, dtype=torch.bfloat16)   # K not a multiple of 8: rows are not 16-byte aligned
    w = _rand(128, 100, seed=2, dtype=torch.bfloat16)
    assert not ops.tc_linear_ok(x, w)
    with pytest.raises(KernelError):
        ops.TensorMap(w, 128)
    with pytest.raises(KernelError):
        ops.TensorMap(_rand(128, 64, seed=3), 128)  # float32


# -------------------------------------------------------- tensor-core attention
@pytest.mark.parametrize("nq,nkv,hd", [(4, 2, 16), (6, 1, 32), (3, 3, 48), (8, 2, 64), (5, 5, 80), (32, 8, 128), (16, 1, 96)])
@pytest.mark.parametrize("window", [0, 70])
def test_attention_decode_mma(nq, nkv, hd, window):
    ops = _ops()
    dt = torch.bfloat16
    lens = [1, 15, 64, 65, 200, 333, 1000]
    k_pool, v_pool, table, ks, vs = _paged(len(lens), lens, nkv, hd, dt, seed=nq * 100 + hd)
    B = len(lens)
    q = _rand(B, nq * hd + 16, seed=41, dtype=dt)[:, : nq * hd]  # rows with a stride of their own
    tok_pos = torch.tensor([l - 1 for l in lens], dtype=torch.int32, device=DEV)
    scale = 1.0 / math.sqrt(hd)
    ref = torch.stack([_attn_ref(q[b].cpu().view(nq, hd), ks[b], vs[b], lens[b] - 1, nq, nkv, scale, window)
                       for b in range(B)]).float()
    plain_out = torch.empty(B, nq * hd, dtype=dt, device=DEV)
    ops.attention_plain(q, plain_out, nq, nkv, hd, k_pool, v_pool, table, 64, tok_pos,
                        torch.arange(B, dtype=torch.int32, device=DEV), scale, window)
    # the pages of all (sequence, head) pairs dealt to one block, to a few (a block then reads several pairs),
    # to about as many as there are pairs, and to more than there are pages (a page each, the rest idle)
    for n_blocks in (1, 3, B * nkv, 29, 64 * nkv):
        out = torch.full((B, nq * hd), float("nan"), dtype=dt, device=DEV)
        scratch = torch.full((ops.attention_decode_scratch(B, nq, nkv, hd, n_blocks),), float("nan"),
                             dtype=torch.float32, device=DEV)
        ops.attention_decode(q, out, scratch, nq, nkv, hd, k_pool, v_pool, table, 64, tok_pos, scale, window, n_blocks)
        torch.testing.assert_close(out.float().cpu().view(B, nq, hd), ref, rtol=2e-2, atol=2e-2)
        torch.testing.assert_close(out.float(), plain_out.float(), rtol=2e-2, atol=2e-2)
        # the kernel's plan is the host's plan of even runs
        host = ops.decode_plan([l - 1 for l in lens], nkv, window, 64, n_blocks, even_only=True)
        assert np.array_equal(ops.attention_decode_plan(tok_pos, nkv, window, n_blocks).cpu().numpy(), host)
        # and with the plan the host likes best (items in equal pieces where the blocks allow) the same comes out
        out2 = torch.full_like(out, float("nan"))
        best = torch.from_numpy(ops.decode_plan([l - 1 for l in lens], nkv, window, 64, n_blocks)).to(DEV)
        ops.attention_decode(q, out2, scratch, nq, nkv, hd, k_pool, v_pool, table, 64, tok_pos, scale, window, n_blocks, best)
        torch.testing.assert_close(out2.float(), plain_out.float(), rtol=2e-2, atol=2e-2)
        ops.check_device_errors(DEV)


@pytest.mark.parametrize("nq,nkv,hd", [(4, 2, 16), (6, 1, 32), (3, 3, 48), (8, 2, 64), (2, 1, 112), (8, 2, 128)])
@pytest.mark.parametrize("window", [0, 70])
def test_attention_prefill_mma(nq, nkv, hd, window):
    ops = _ops()
    dt = torch.bfloat16
    # (cached before, new now) per sequence: whole prompts, a continued chunk, a single token
    spans = [(0, 1), (0, 63), (0, 64), (0, 130), (100, 77), (64, 64), (199, 1), (5, 200)]
    lens = [s + n for s, n in spans]
    k_pool, v_pool, table, ks, vs = _paged(len(lens), lens, nkv, hd, dt, seed=nq * 7 + hd)
    tok_pos, tok_seq, tile_seq, tile_tok0, tile_rows = [], [], [], [], []
    for b, (s, n) in enumerate(spans):
        for j in range(0, n, 64):
            tile_seq.append(b); tile_tok0.append(len(tok_pos) + j); tile_rows.append(min(64, n - j))
        tok_pos += list(range(s, s + n)); tok_seq += [b] * n
    T = len(tok_pos)
    q = _rand(T, nq * hd, seed=43, dtype=dt)
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=DEV)
    scale = 1.0 / math.sqrt(hd)
    out = torch.full((T, nq * hd), float("nan"), dtype=dt, device=DEV)
    ops.attention_prefill(q, out, nq, nkv, hd, k_pool, v_pool, table, 64, i32(tok_pos), i32(tile_seq), i32(tile_tok0),
                          i32(tile_rows), scale, window)
    plain_out = torch.empty_like(out)
    ops.attention_plain(q, plain_out, nq, nkv, hd, k_pool, v_pool, table, 64, i32(tok_pos), i32(tok_seq), scale, window)
    torch.testing.assert_close(out.float(), plain_out.float(), rtol=2e-2, atol=2e-2)
    for i in (0, 1, 63, 64, 64 + 129, T - 1, T - 200, T - 137):
        ref = _attn_ref(q[i].cpu().view(nq, hd), ks[tok_seq[i]], vs[tok_seq[i]], tok_pos[i], nq, nkv, scale, window)
        torch.testing.assert_close(out[i].float().cpu().view(nq, hd), ref.float(), rtol=2e-2, atol=2e-2)


@pytest.mark.parametrize("nq,nkv,window", [(2, 1, 0), (4, 2, 0), (12, 2, 0), (16, 2, 130), (8, 8, 0), (6, 2, 0)])
def test_attention_prefill_tcgen05_against_mma_sync_and_plain(nq, nkv, window):
    """Heads of 128 with an even group run on the tcgen05 kernel (two heads a block, P V with V as it
    lies in the cache); odd groups and (8, 8) stay on mma.sync.  Both against the plain kernel, on
    prompts that start inside a page, end inside one, continue a cached prefix, and a lone token."""
    ops = _ops()
    dt, hd = torch.bfloat16, 128
    spans = [(0, 200), (37, 64), (0, 1), (64, 129), (250, 70), (3, 5)]
    lens = [s + n for s, n in spans]
    k_pool, v_pool, table, ks, vs = _paged(len(lens), lens, nkv, hd, dt, seed=nq * 3 + nkv)
    tok_pos, tok_seq, tile_seq, tile_tok0, tile_rows = [], [], [], [], []
    for b, (s0, n) in enumerate(spans):
        for j in range(0, n, 64):
            tile_seq.append(b); tile_tok0.append(len(tok_pos) + j); tile_rows.append(min(64, n - j))
        tok_pos += list(range(s0, s0 + n)); tok_seq += [b] * n
    T = len(tok_pos)
    q = _rand(T, nq * hd, seed=44, dtype=dt)
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=DEV)
    scale = 1.0 / math.sqrt(hd)
    args = (nq, nkv, hd, k_pool, v_pool, table, 64, i32(tok_pos), i32(tile_seq), i32(tile_tok0), i32(tile_rows), scale, window)
    outs = {}
    for tc in (True, False):
        out = torch.full((T, nq * hd), float("nan"), dtype=dt, device=DEV)
        before = dict(ops.LAUNCHES_BY_MODULE)
        ops.attention_prefill(q, out, *args, tcgen05=tc)
        made = {m: n - before.get(m, 0) for m, n in ops.LAUNCHES_BY_MODULE.items() if n != before.get(m, 0)}
        tc_takes_it = (nq // nkv) % 2 == 0
        assert made == ({"attention_tc": 1} if tc and tc_takes_it else {"attention_mma": 1}), made
        outs[tc] = out
    plain_out = torch.empty_like(outs[True])
    ops.attention_plain(q, plain_out, nq, nkv, hd, k_pool, v_pool, table, 64, i32(tok_pos), i32(tok_seq), scale, window)
    for out in outs.values():
        assert torch.isfinite(out.float()).all()
        torch.testing.assert_close(out.float(), plain_out.float(), rtol=2e-2, atol=2e-2)
    for i in (0, 199, 200, 263, T - 1, T - 6, T - 75):
        ref = _attn_ref(q[i].cpu().view(nq, hd), ks[tok_seq[i]], vs[tok_seq[i]], tok_pos[i], nq, nkv, scale, window)
        torch.testing.assert_close(outs[True][i].float().cpu().view(nq, hd), ref.float(), rtol=2e-2, atol=2e-2)
    ops.check_device_errors(DEV)


def test_attention_prefill_tcgen05_finds_one_far_key_and_respects_the_causal_edge():
    """One key far back that dominates, and keys just past each row's own position that would dominate
    if they were seen: the tcgen05 kernel's masks and its lazily rescaled accumulator."""
    ops = _ops()
    dt, nq, nkv, hd, L = torch.bfloat16, 4, 2, 128, 700
    k_pool, v_pool, table, ks, vs = _paged(1, [L], nkv, hd, dt, seed=9)
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=DEV)
    start = L - 150  # the last 150 tokens are new
    tok_pos = list(range(start, L))
    tile_seq, tile_tok0, tile_rows = [0, 0, 0], [0, 64, 128], [64, 64, 22]
    q = _rand(len(tok_pos), nq * hd, seed=13, dtype=dt)
    scale = 1.0 / math.sqrt(hd)
    for target in (3, 63, 64, start - 1, start + 70):
        kp = k_pool.clone()
        page, off = int(table[0, target // 64]), target % 64
        kp[page, :, off, :] = 6.0 * torch.sign(q[-1].view(nq, hd)[0]).to(dt)  # every query head leans on this key
        out = torch.empty(len(tok_pos), nq * hd, dtype=dt, device=DEV)
        ops.attention_prefill(q, out, nq, nkv, hd, kp, v_pool, table, 64, i32(tok_pos), i32(tile_seq), i32(tile_tok0),
                              i32(tile_rows), scale, 0)
        plain_out = torch.empty_like(out)
        ops.attention_plain(q, plain_out, nq, nkv, hd, kp, v_pool, table, 64, i32(tok_pos), i32([0] * len(tok_pos)), scale, 0)
        torch.testing.assert_close(out.float(), plain_out.float(), rtol=2e-2, atol=2e-2)
        # rows before the target (when it is a new token) must not have seen it
        if target >= start:
            row = target - start - 1
            assert (out[row].float() - plain_out[row].float()).abs().max().item() < 2e-2
    ops.check_device_errors(DEV)


def test_attention_mma_finds_one_far_key():
    ops = _ops()
    dt = torch.bfloat16
    nq, nkv, hd, L = 8, 2, 128, 1500
    k_pool, v_pool, table, ks, vs = _paged(1, [L], nkv, hd, dt, seed=5)
    q = _rand(1, nq * hd, seed=12, dtype=dt)
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=DEV)
    for target in (0, 15, 16, 63, 64, 700, L - 2, L - 1):
        kp = k_pool.clone()
        page, off = int(table[0, target // 64]), target % 64
        for kvh in range(nkv):
            qh = q[0].view(nq, hd)[kvh * 4 + 1].float()
            kp[page, kvh, off] = (qh / qh.norm() * 60.0).to(dt)
        for mode in ("decode", "prefill"):
            out = torch.empty(1, nq * hd, dtype=dt, device=DEV)
            if mode == "decode":
                scratch = torch.empty(ops.attention_decode_scratch(1, nq, nkv, hd, 10), dtype=torch.float32, device=DEV)
                ops.attention_decode(q, out, scratch, nq, nkv, hd, kp, v_pool, table, 64, i32([L - 1]), 1.0, 0, 10)
            else:
                ops.attention_prefill(q, out, nq, nkv, hd, kp, v_pool, table, 64, i32([L - 1]), i32([0]), i32([0]),
                                      i32([1]), 1.0, 0)
            for kvh in range(nkv):
                got = out[0].view(nq, hd)[kvh * 4 + 1].float().cpu()
                torch.testing.assert_close(got, vs[0][target, kvh].float(), rtol=2e-2, atol=2e-2)


def test_prep_takes_32_bit_rows_and_writes_bfloat16():
    """Few tokens: the product leaves 32-bit rows; queries and cache are bfloat16."""
    ops = _ops()
    nq, nkv, hd, T = 4, 2, 32, 5
    width = (nq + 2 * nkv) * hd
    whole = _rand(T, width, seed=61)
    qn, kn = 1 + 0.2 * _rand(hd, seed=62), 1 + 0.2 * _rand(hd, seed=63)
    freqs, _ = plain.rope_frequencies(hd, 10000.0)
    ang = (torch.arange(100, dtype=torch.float32)[:, None] * freqs[None, :]).double()
    cos, sin = torch.cos(ang).float().to(DEV), torch.sin(ang).float().to(DEV)
    pos = torch.tensor([0, 1, 64, 65, 3], dtype=torch.int32, device=DEV)
    seq = torch.tensor([0, 0, 0, 0, 1], dtype=torch.int32, device=DEV)
    table = torch.tensor([[1, 2], [0, 3]], dtype=torch.int32, device=DEV)
    res = []
    for src in (whole, whole.to(torch.bfloat16)):
        kp = torch.zeros(4, nkv, 64, hd, dtype=torch.bfloat16, device=DEV)
        vp = torch.zeros_like(kp)
        q = torch.zeros(T, nq * hd, dtype=torch.bfloat16, device=DEV)
        ops.qk_norm_rope_cache(src, 0, nq * hd, (nq + nkv) * hd, nq, nkv, hd, qn, kn, 1e-6, cos, sin, hd, pos, seq,
                               kp, vp, table, 64, q_out=q)
        res.append((q, kp, vp))
    for a, b in zip(res[0], res[1]):  # from 32-bit rows against from the rounded rows: bf16 apart at most
        torch.testing.assert_close(a.float(), b.float(), rtol=2e-2, atol=2e-2)
    assert res[0][0].abs().sum() > 0 and res[0][1].abs().sum() > 0


# ----------------------------------------------- few tokens: the weight-streaming product
@pytest.mark.parametrize("m,n,k,rows,kkb,splits,kstack", [
    (1, 128, 64, 128, 1, 1, 1), (8, 4096, 4096, 56, 2, 2, 1), (5, 1000, 264, 8, 1, 1, 1), (16, 300, 1032, 24, 1, 3, 1),
    (11, 132, 8192, 16, 2, 8, 1), (33, 520, 704, 104, 2, 2, 1), (64, 392, 512, 40, 4, 2, 1), (64, 392, 520, 40, 1, 5, 1),
    (8, 4096, 12288, 112, 2, 4, 1), (3, 200, 1536, 72, 3, 4, 1),
    (8, 4096, 4096, 32, 8, 1, 4), (8, 6144, 4096, 48, 6, 1, 2), (16, 300, 1088, 24, 10, 1, 5), (1, 100, 704, 8, 16, 1, 16),
    (33, 520, 704, 40, 6, 1, 3), (64, 392, 1536, 32, 4, 1, 4), (50, 200, 960, 56, 4, 1, 2), (8, 4096, 12288, 32, 8, 1, 4),
    # 65 to 128 tokens: the widest token tile, plain and with K cut into a cluster
    (128, 4096, 4096, 128, 1, 4, 1), (100, 520, 1088, 104, 1, 3, 1), (65, 392, 512, 40, 1, 2, 1), (128, 264, 320, 88, 1, 1, 1),
    (97, 4096, 12288, 128, 1, 4, 1), (127, 132, 1024, 16, 1, 8, 1)])
def test_gemm_tc_rows_store_accumulate_gated(m, n, k, rows, kkb, splits, kstack):
    """Every epilogue of the weight-streaming product against float64, at tile heights that
    divide nothing (the last block's rows run past the matrix), K cut into clusters of
    splits of unequal length, boxes of one to sixteen K blocks, and K blocks stacked into
    one MMA (with a last box that runs past K)."""
    ops = _ops()
    from skyla_kernel_b200.parts.feedforward import fuse_gate_up
    x = _rand(m, k, seed=91, dtype=torch.bfloat16)
    w = _rand(n, k, seed=92, dtype=torch.bfloat16, scale=0.1)
    ref = x.double() @ w.double().T
    tol = dict(rtol=1e-2, atol=1e-2 * ref.abs().max().item())
    wm = ops.TensorMap(w, rows, kkb)
    y = torch.full((m, n), float("nan"), device=DEV)
    ops.gemm_tc_rows(x, wm, rows, n, y, ops.TC_STORE_F32, kkb=kkb, splits=splits, kstack=kstack)
    assert (y.double() - ref).abs().max().item() <= 2e-5 * ref.abs().max().item() + 1e-6  # float32 sums of exact products
    yb = torch.empty(m, n, dtype=torch.bfloat16, device=DEV)
    ops.gemm_tc_rows(x, wm, rows, n, yb, ops.TC_STORE_BF16, kkb=kkb, splits=splits, kstack=kstack)
    torch.testing.assert_close(yb.double(), ref, **tol)
    base = _rand(m, n, seed=93)
    acc = base.clone()
    ops.gemm_tc_rows(x, wm, rows, n, acc, ops.TC_ACCUM_F32, kkb=kkb, splits=splits, kstack=kstack)
    ops.gemm_tc_rows(x, wm, rows, n, acc, ops.TC_ACCUM_F32, kkb=kkb, splits=splits, kstack=kstack)
    assert (acc.double() - (base.double() + 2 * ref)).abs().max().item() <= 1e-4 * ref.abs().max().item() + 1e-5
    g, u = _rand(n, k, seed=94, dtype=torch.bfloat16, scale=0.1), _rand(n, k, seed=95, dtype=torch.bfloat16, scale=0.1)
    act = torch.empty(m, n, dtype=torch.bfloat16, device=DEV)
    kkb = min(kkb, 2)  # the gated product brings two tiles per K block
    ops.gemm_tc_rows(x, ops.TensorMap(fuse_gate_up(g, u), rows, kkb), rows, n, act, ops.TC_GLU_BF16, kkb=kkb)
    gd, ud = x.double() @ g.double().T, x.double() @ u.double().T
    ref_act = gd / (1 + torch.exp(-gd)) * ud
    torch.testing.assert_close(act.double(), ref_act, rtol=1e-2, atol=1e-2 * ref_act.abs().max().item())
    ops.check_device_errors(DEV)


@pytest.mark.parametrize("m,n,k,rows,kkb,kstack,n2,rows2,kkb2,kstack2", [
    (8, 4096, 4096, 32, 8, 4, 6144, 48, 6, 2), (5, 264, 520, 24, 1, 1, 200, 72, 1, 1), (16, 328, 704, 40, 6, 3, 136, 8, 16, 16),
    (1, 128, 64, 128, 1, 1, 128, 128, 1, 1), (11, 1000, 1536, 56, 4, 2, 520, 88, 2, 1),
    # K cut into a cluster of splits on either side (kstack = -splits): 17 to 64 tokens are served so
    (64, 4096, 4096, 128, 2, -4, 6144, 96, 2, -2), (40, 520, 1088, 104, 1, -3, 200, 72, 2, -2), (17, 328, 704, 40, 2, -2, 136, 128, 1, -3),
    (3, 264, 640, 24, 1, -4, 264, 24, 1, -5),
    (128, 4096, 4096, 128, 1, -4, 6144, 96, 1, -2), (70, 520, 1088, 104, 1, -3, 200, 72, 1, -2), (99, 328, 704, 40, 1, 1, 136, 128, 1, 1)])
def test_gemm_tc_rows_norm_ahead_then_scale_in(m, n, k, rows, kkb, kstack, n2, rows2, kkb2, kstack2):
    """x += a W^T leaves x * norm weight in bfloat16 and the blocks' shares of the rows' sums of
    squares; the next product takes those and must equal the product of rmsnorm(x)."""
    ops = _ops()
    splits = splits2 = 1
    if kstack < 0:
        splits, kstack = -kstack, 1
    if kstack2 < 0:
        splits2, kstack2 = -kstack2, 1
    from skyla_kernel_b200.parts.feedforward import fuse_gate_up
    a = _rand(m, k, seed=61, dtype=torch.bfloat16)
    w = _rand(n, k, seed=62, dtype=torch.bfloat16, scale=0.1)
    x0 = _rand(m, n, seed=63, scale=1.5)
    nw = 1 + 0.2 * _rand(n, seed=64)
    x = x0.clone()
    blocks = -(-n // rows)
    xw = torch.full((m, n), float("nan"), dtype=torch.bfloat16, device=DEV)
    shares = torch.full((blocks, m), float("nan"), device=DEV)
    ops.gemm_tc_rows(a, ops.TensorMap(w, rows, kkb), rows, n, x, ops.TC_ACCUM_F32, kkb=kkb, kstack=kstack, splits=splits,
                     norm_ahead=(nw, xw, shares))
    want_x = x0.double() + a.double() @ w.double().T
    assert (x.double() - want_x).abs().max().item() <= 1e-5 * want_x.abs().max().item() + 1e-6
    assert torch.equal(xw, (x * nw).to(torch.bfloat16))                       # the very rows that were stored
    ssq = shares.double().sum(0)
    torch.testing.assert_close(ssq, (x.double() ** 2).sum(1), rtol=1e-5, atol=1e-6)
    # the next product: plain, and gated
    eps = 1e-5
    h = plain.rmsnorm(x.double().cpu(), nw.double().cpu(), eps)
    w2 = _rand(n2, n, seed=65, dtype=torch.bfloat16, scale=0.1)
    ref = h @ w2.double().cpu().T
    y = torch.full((m, n2), float("nan"), device=DEV)
    ops.gemm_tc_rows(xw, ops.TensorMap(w2, rows2, kkb2 if n % 64 == 0 else 1), rows2, n2, y, ops.TC_STORE_F32,
                     kkb=kkb2 if n % 64 == 0 else 1, kstack=kstack2 if n % 64 == 0 else 1, splits=splits2,
                     scale_in=(shares, eps))
    torch.testing.assert_close(y.double().cpu(), ref, rtol=2e-2, atol=2e-2 * ref.abs().max().item())
    assert (y.double().cpu() - ref).abs().mean().item() < 4e-3 * ref.abs().max().item()
    g, u = _rand(n2, n, seed=66, dtype=torch.bfloat16, scale=0.1), _rand(n2, n, seed=67, dtype=torch.bfloat16, scale=0.1)
    act = torch.empty(m, n2, dtype=torch.bfloat16, device=DEV)
    kk = min(2, kkb2) if n % 64 == 0 else 1
    ops.gemm_tc_rows(xw, ops.TensorMap(fuse_gate_up(g, u), rows2, kk), rows2, n2, act, ops.TC_GLU_BF16, kkb=kk,
                     scale_in=(shares, eps))
    gd, ud = h @ g.double().cpu().T, h @ u.double().cpu().T
    ref_act = gd / (1 + torch.exp(-gd)) * ud
    torch.testing.assert_close(act.double().cpu(), ref_act, rtol=3e-2, atol=3e-2 * ref_act.abs().max().item())
    ops.check_device_errors(DEV)


def test_rows_plan_fills_the_sms():
    ops = _ops()
    for n, k, gated in [(6144, 4096, False), (4096, 4096, False), (12288, 4096, True), (4096, 12288, False),
                        (151936, 4096, False), (96, 80, False), (160, 80, True), (25600, 5120, True), (2560, 9728, False)]:
        for bn in (16, 32, 64):
            rows, splits, kkb, kstack = ops.rows_plan(n, k, gated, bn)
            assert rows % 8 == 0 and 8 <= rows <= 128 and splits == 1 and kkb % kstack == 0 and 1 <= kkb <= 16
            assert kstack * rows <= 128 and kstack * bn <= 256 and (kkb == 1 or k % 64 == 0) and (kstack == 1 or not gated)
            blocks = -(-n // rows)
            assert n < 148 * 8 or blocks / (-(-blocks // 148) * 148) >= 0.7  # the waves are nearly full
            stage = kkb * (rows * (2 if gated else 1) + bn) * 128
            assert 2 * stage + 40 * 1024 <= 212 * 1024  # at least two stages beside the epilogue's room


def test_gemm_tc_rows_refuses():
    ops = _ops()
    from skyla_kernel_b200.kernels import KernelError
    x = _rand(130, 64, seed=1, dtype=torch.bfloat16)
    w = _rand(128, 64, seed=2, dtype=torch.bfloat16)
    with pytest.raises(KernelError):  # too many tokens
        ops.gemm_tc_rows(x, ops.TensorMap(w, 128), 128, 128, torch.empty(130, 128, device=DEV), ops.TC_STORE_F32)
    with pytest.raises(KernelError):  # K blocks are stacked for token tiles up to 64
        ops.gemm_tc_rows(_rand(100, 256, seed=6, dtype=torch.bfloat16), ops.TensorMap(_rand(128, 256, seed=7, dtype=torch.bfloat16), 64, 2),
                         64, 128, torch.empty(100, 128, device=DEV), ops.TC_STORE_F32, kkb=2, kstack=2)
    with pytest.raises(KernelError):  # a tile height that is no multiple of 8
        ops.gemm_tc_rows(x[:4], ops.TensorMap(w, 100), 100, 128, torch.empty(4, 128, device=DEV), ops.TC_STORE_F32)
    with pytest.raises(KernelError):  # an epilogue it does not have
        ops.gemm_tc_rows(x[:4], ops.TensorMap(w, 128), 128, 128, torch.empty(4, 128, device=DEV), 4)
    with pytest.raises(KernelError):  # more splits than K blocks
        ops.gemm_tc_rows(x[:4], ops.TensorMap(w, 128), 128, 128, torch.empty(4, 128, device=DEV), ops.TC_STORE_F32, splits=2)
    with pytest.raises(KernelError, match="outputs in fours"):  # K splits of a width that is no multiple of four
        ops.gemm_tc_rows(_rand(4, 256, seed=4, dtype=torch.bfloat16), ops.TensorMap(_rand(130, 256, seed=5, dtype=torch.bfloat16), 128),
                         128, 130, torch.empty(4, 130, device=DEV), ops.TC_STORE_F32, splits=2)
    with pytest.raises(KernelError):  # boxes of several K blocks over a width that is no multiple of 64
        ops.TensorMap(_rand(128, 72, seed=3, dtype=torch.bfloat16), 128, 2)


@pytest.mark.parametrize("nq,nkv,hd,n_rot,window", [(32, 8, 128, 128, 0), (6, 1, 32, 32, 0), (3, 3, 48, 24, 70), (8, 2, 64, 64, 0)])
def test_attention_decode_fused_prep(nq, nkv, hd, n_rot, window):
    """The decode kernel finishing q, k and v itself against prep kernel + decode kernel."""
    ops = _ops()
    dt = torch.bfloat16
    lens = [1, 64, 65, 200, 333, 128]   # lengths after the new token
    B = len(lens)
    width = (nq + 2 * nkv) * hd
    k_pool, v_pool, table, ks, vs = _paged(B, lens, nkv, hd, dt, seed=nq + hd)
    rows = _rand(B, width, seed=101)
    qn, kn = 1 + 0.2 * _rand(hd, seed=103), 1 + 0.2 * _rand(hd, seed=104)
    freqs, _ = plain.rope_frequencies(n_rot, 10000.0)
    ang = (torch.arange(512, dtype=torch.float32)[:, None] * freqs[None, :]).double()
    cos, sin = torch.cos(ang).float().to(DEV), torch.sin(ang).float().to(DEV)
    tok_pos = torch.tensor([l - 1 for l in lens], dtype=torch.int32, device=DEV)
    seq = torch.arange(B, dtype=torch.int32, device=DEV)
    scale = 1.0 / math.sqrt(hd)
    n_blocks = 3 * nkv + 1
    plan = torch.from_numpy(ops.decode_plan([l - 1 for l in lens], nkv, window, 64, n_blocks)).to(DEV)
    # two kernels
    kp1, vp1 = k_pool.clone(), v_pool.clone()
    q = torch.empty(B, nq * hd, dtype=dt, device=DEV)
    ops.qk_norm_rope_cache(rows, 0, nq * hd, (nq + nkv) * hd, nq, nkv, hd, qn, kn, 1e-6, cos, sin, n_rot, tok_pos, seq,
                           kp1, vp1, table, 64, q_out=q)
    want = torch.empty(B, nq * hd, dtype=dt, device=DEV)
    scratch = torch.empty(ops.attention_decode_scratch(B, nq, nkv, hd, n_blocks), dtype=torch.float32, device=DEV)
    ops.attention_decode(q, want, scratch, nq, nkv, hd, kp1, vp1, table, 64, tok_pos, scale, window, n_blocks, plan)
    # one kernel
    kp2, vp2 = k_pool.clone(), v_pool.clone()
    got = torch.full_like(want, float("nan"))
    ops.attention_decode_fused(rows, 0, nq * hd, (nq + nkv) * hd, qn, kn, 1e-6, cos, sin, n_rot, got,
                               scratch, nq, nkv, hd, kp2, vp2, table, 64, tok_pos, scale, window, n_blocks, plan)
    torch.testing.assert_close(got.float(), want.float(), rtol=2e-2, atol=2e-2)
    assert torch.equal(kp2, kp1) and torch.equal(vp2, vp1)  # the same k and v reached the cache
    assert not torch.equal(kp2, k_pool)


# ---------------------------------------------------------------- the prompt kernel (tokens are the tile's rows)
@pytest.mark.parametrize("m,n,k,cut", [
    (129, 256, 64, False), (130, 384, 1032, True), (300, 200, 264, False), (257, 203, 96, False), (1000, 640, 512, False),
    (128, 1000, 328, False), (300, 512, 12800, True), (1280, 4096, 6400, False), (700, 1000, 4104, True), (70, 2048, 4096, True)])
def test_gemm_prompt_store_accumulate_gated(m, n, k, cut):
    """Where ``cut``, the tiles are few and are cut along K over several blocks, whose accumulators
    meet in the block that has the tile's first K blocks; elsewhere whole tiles."""
    ops = _ops()
    if torch.cuda.get_device_properties(DEV).multi_processor_count == 148:
        assert (ops.prompt_cut_blocks(m, n, k, False, DEV) > 0) == cut
    from skyla_kernel_b200.parts.feedforward import fuse_gate_up
    x = _rand(m, k, seed=71, dtype=torch.bfloat16)
    w = _rand(n, k, seed=72, dtype=torch.bfloat16, scale=0.1)
    ref = x.double() @ w.double().T
    scale = ref.abs().max().item() * max(1.0, k / 4096)  # rounding of a 32-bit running sum grows with its length
    wm = ops.TensorMap(w, 128)
    y32 = torch.full((m, n), float("nan"), dtype=torch.float32, device=DEV)
    ops.gemm_prompt(x, wm, n, y32, ops.TC_STORE_F32)
    assert (y32.double() - ref).abs().max().item() <= 2e-5 * scale + 1e-6
    y16 = torch.empty(m, n, dtype=torch.bfloat16, device=DEV)
    ops.gemm_prompt(x, wm, n, y16, ops.TC_STORE_BF16)
    assert torch.equal(y16, y32.to(torch.bfloat16))
    acc = _rand(m, n, seed=73)
    before = acc.clone()
    ops.gemm_prompt(x, wm, n, acc, ops.TC_ACCUM_F32)
    assert (acc.double() - before.double() - ref).abs().max().item() <= 2e-5 * scale + 1e-5
    again = before.clone()
    ops.gemm_prompt(x, wm, n, again, ops.TC_ACCUM_F32)
    assert torch.equal(again, acc)  # shares are added in block order: the same bits every time
    # rows of a wider buffer: what lies beside them stays
    wide = torch.full((m, n + 24), 7.0, dtype=torch.float32, device=DEV)
    ops.gemm_prompt(x, wm, n, wide[:, 8:8 + n], ops.TC_STORE_F32)
    assert torch.equal(wide[:, 8:8 + n], y32) and (wide[:, :8] == 7).all() and (wide[:, 8 + n:] == 7).all()
    g, u = _rand(n, k, seed=74, dtype=torch.bfloat16, scale=0.2), _rand(n, k, seed=75, dtype=torch.bfloat16, scale=0.2)
    fused = fuse_gate_up(g, u)
    act = torch.empty(m, n, dtype=torch.bfloat16, device=DEV)
    ops.gemm_prompt(x, ops.TensorMap(fused, 128), n, act, ops.TC_GLU_BF16)
    gd, ud = x.double() @ g.double().T, x.double() @ u.double().T
    ref_act = gd / (1 + torch.exp(-gd)) * ud
    torch.testing.assert_close(act.double(), ref_act, rtol=1e-2, atol=1e-2 * ref_act.abs().max().item())
    plain_act = torch.empty_like(act)
    ops.linear_plain(x, fused, plain_act, ops.GATED)
    torch.testing.assert_close(act.float(), plain_act.float(), rtol=2e-2, atol=1e-3 * max(1.0, k / 512))
    ops.check_device_errors(DEV)
    assert int(ops.default_state(DEV).prompt_shares()[1].abs().sum()) == 0  # every share that was left was taken


@pytest.mark.parametrize("m,n,k,n2", [(300, 512, 264, 384), (129, 264, 520, 200), (515, 1000, 128, 136), (300, 512, 12800, 384)])
def test_gemm_prompt_norm_ahead_then_scale_in(m, n, k, n2):
    """x += a W^T leaves x * norm weight in bfloat16 and the tiles' shares of the rows' sums of
    squares; the next product takes those and must equal the product of rmsnorm(x)."""
    ops = _ops()
    from skyla_kernel_b200.parts.feedforward import fuse_gate_up
    a = _rand(m, k, seed=81, dtype=torch.bfloat16)
    w = _rand(n, k, seed=82, dtype=torch.bfloat16, scale=0.1)
    x0 = _rand(m, n, seed=83, scale=1.5)
    nw = 1 + 0.2 * _rand(n, seed=84)
    x = x0.clone()
    parts = ops.prompt_ahead_parts(n)
    xw = torch.full((m, n), float("nan"), dtype=torch.bfloat16, device=DEV)
    shares = torch.full((parts, m), float("nan"), device=DEV)
    ops.gemm_prompt(a, ops.TensorMap(w, 128), n, x, ops.TC_ACCUM_F32, norm_ahead=(nw, xw, shares))
    want_x = x0.double() + a.double() @ w.double().T
    assert (x.double() - want_x).abs().max().item() <= 1e-5 * max(1.0, k / 4096) * want_x.abs().max().item() + 1e-6
    assert torch.equal(xw, (x * nw).to(torch.bfloat16))  # the very rows that were stored
    torch.testing.assert_close(shares.double().sum(0), (x.double() ** 2).sum(1), rtol=1e-5, atol=1e-6)
    eps = 1e-5
    h = plain.rmsnorm(x.double().cpu(), nw.double().cpu(), eps)
    w2 = _rand(n2, n, seed=85, dtype=torch.bfloat16, scale=0.1)
    ref = h @ w2.double().cpu().T
    y = torch.full((m, n2), float("nan"), device=DEV)
    ops.gemm_prompt(xw, ops.TensorMap(w2, 128), n2, y, ops.TC_STORE_F32, scale_in=(shares, eps))
    torch.testing.assert_close(y.double().cpu(), ref, rtol=2e-2, atol=2e-2 * ref.abs().max().item())
    assert (y.double().cpu() - ref).abs().mean().item() < 4e-3 * ref.abs().max().item()
    g, u = _rand(n2, n, seed=86, dtype=torch.bfloat16, scale=0.1), _rand(n2, n, seed=87, dtype=torch.bfloat16, scale=0.1)
    act = torch.empty(m, n2, dtype=torch.bfloat16, device=DEV)
    ops.gemm_prompt(xw, ops.TensorMap(fuse_gate_up(g, u), 128), n2, act, ops.TC_GLU_BF16, scale_in=(shares, eps))
    gd, ud = h @ g.double().cpu().T, h @ u.double().cpu().T
    ref_act = gd / (1 + torch.exp(-gd)) * ud
    torch.testing.assert_close(act.double().cpu(), ref_act, rtol=3e-2, atol=3e-2 * ref_act.abs().max().item())
    # shares left by the weight-streaming kernel are taken just as well (a producer of few rows, then many: not in
    # one step, but the contract is the same): shares summed in another cut give the same scalars
    one = shares.sum(0, keepdim=True).contiguous()
    y1 = torch.empty_like(y)
    ops.gemm_prompt(xw, ops.TensorMap(w2, 128), n2, y1, ops.TC_STORE_F32, scale_in=(one, eps))
    torch.testing.assert_close(y1, y, rtol=1e-5, atol=1e-6)
    ops.check_device_errors(DEV)


@pytest.mark.parametrize("nq,nkv,hd,use_norm,use_rope,scaled,k", [
    (4, 2, 128, True, True, True, 264), (5, 1, 64, True, True, False, 264), (3, 3, 32, False, True, False, 264),
    (2, 1, 256, True, False, True, 264), (6, 2, 128, False, False, False, 264), (4, 2, 128, True, True, True, 12800),
    (5, 1, 64, True, True, False, 2048)])
def test_gemm_prompt_finishes_heads_into_queries_and_cache(nq, nkv, hd, use_norm, use_rope, scaled, k):
    """The q/k/v product whose epilogue norms and rotates the heads and writes k and v into the
    paged cache, against the plain steps on a float64 product; positions that start late in a
    sequence, two sequences, shuffled pages."""
    ops = _ops()
    lens, starts = [150, 70], [37, 64]  # new tokens of each sequence and the position of its first
    T = sum(lens)
    positions = [s + i for l, s in zip(lens, starts) for i in range(l)]
    seqs = [b for b, l in enumerate(lens) for _ in range(l)]
    g = torch.Generator().manual_seed(5)
    table = torch.randperm(9, generator=g)[:8].view(2, 4).to(torch.int32).to(DEV)
    n = (nq + 2 * nkv) * hd
    x = _rand(T, k, seed=91, dtype=torch.bfloat16)
    w = _rand(n, k, seed=92, dtype=torch.bfloat16, scale=0.1)
    qn, kn = 1 + 0.2 * _rand(hd, seed=93), 1 + 0.2 * _rand(hd, seed=94)
    freqs, _ = plain.rope_frequencies(hd, 10000.0)
    ang = (torch.arange(300, dtype=torch.float32)[:, None] * freqs[None, :]).double()
    cos, sin = torch.cos(ang).float().to(DEV), torch.sin(ang).float().to(DEV)
    k_pool = torch.zeros(9, nkv, 64, hd, dtype=torch.bfloat16, device=DEV)
    v_pool = torch.zeros_like(k_pool)
    q_out = torch.full((T, nq * hd), float("nan"), dtype=torch.bfloat16, device=DEV)
    shares, eps_in = None, 1e-5
    if scaled:
        shares = (0.5 + torch.rand(3, T, generator=g)).to(DEV)
    ops.gemm_prompt(x, ops.TensorMap(w, 128), n, q_out, ops.TC_QKV_PREP,
                    scale_in=(shares, eps_in) if scaled else None,
                    prep=dict(nq=nq, nkv=nkv, hd=hd, q_norm=qn if use_norm else None, k_norm=kn if use_norm else None,
                              eps=1e-6, cos=cos if use_rope else None, sin=sin if use_rope else None,
                              tok_pos=torch.tensor(positions, dtype=torch.int32, device=DEV),
                              tok_slot=torch.tensor(seqs, dtype=torch.int32, device=DEV),
                              k_pool=k_pool, v_pool=v_pool, page_table=table, page_size=64))
    ops.check_device_errors(DEV)
    o = (x.double() @ w.double().T).cpu()
    if scaled:
        o = o * (1.0 / torch.sqrt(shares.double().cpu().sum(0) / k + eps_in))[:, None]
    pos_t = torch.tensor(positions)
    q = o[:, : nq * hd].reshape(T, nq, hd)
    kk = o[:, nq * hd:(nq + nkv) * hd].reshape(T, nkv, hd)
    v = o[:, (nq + nkv) * hd:].reshape(T, nkv, hd)
    if use_norm:
        q, kk = plain.rmsnorm(q, qn.double().cpu(), 1e-6), plain.rmsnorm(kk, kn.double().cpu(), 1e-6)
    if use_rope:
        q, kk = plain.rope_neox(q, pos_t, freqs, 1.0, hd), plain.rope_neox(kk, pos_t, freqs, 1.0, hd)
    tol = dict(rtol=1e-2, atol=1e-2 * float(max(q.abs().max(), kk.abs().max(), v.abs().max())))
    torch.testing.assert_close(q_out.double().cpu().view(T, nq, hd), q.double(), **tol)
    pages = table.cpu()[torch.tensor(seqs), pos_t // 64].long()
    torch.testing.assert_close(k_pool.cpu()[pages, :, pos_t % 64].double(), kk.double(), **tol)
    torch.testing.assert_close(v_pool.cpu()[pages, :, pos_t % 64].double(), v.double(), **tol)
    mask = torch.ones(9, 64, dtype=torch.bool)
    mask[pages, pos_t % 64] = False
    assert (k_pool.float().cpu().abs().sum((1, 3))[mask] == 0).all()  # nothing else was written
    assert (v_pool.float().cpu().abs().sum((1, 3))[mask] == 0).all()
    # and the same numbers as the two-kernel path leaves, beyond its extra rounding of the product
    qkv = torch.empty(T, n, dtype=torch.bfloat16, device=DEV)
    ops.gemm_prompt(x, ops.TensorMap(w, 128), n, qkv, ops.TC_STORE_BF16, scale_in=(shares, eps_in) if scaled else None)
    k2, v2 = torch.zeros_like(k_pool), torch.zeros_like(v_pool)
    ops.qk_norm_rope_cache(qkv, 0, nq * hd, (nq + nkv) * hd, nq, nkv, hd, qn if use_norm else None,
                           kn if use_norm else None, 1e-6, cos if use_rope else None, sin if use_rope else None, hd,
                           torch.tensor(positions, dtype=torch.int32, device=DEV),
                           torch.tensor(seqs, dtype=torch.int32, device=DEV), k2, v2, table, 64)
    torch.testing.assert_close(q_out.float(), qkv[:, : nq * hd].float(), rtol=3e-2, atol=3e-2 * tol["atol"] / 1e-2)
    torch.testing.assert_close(k_pool.float(), k2.float(), rtol=3e-2, atol=3e-2 * tol["atol"] / 1e-2)
    assert torch.equal(v_pool, v2)


def test_gemm_prompt_refuses():
    ops = _ops()
    from skyla_kernel_b200.kernels import KernelError
    x = _rand(200, 64, seed=95, dtype=torch.bfloat16)
    w = _rand(6 * 48, 64, seed=96, dtype=torch.bfloat16)
    wm = ops.TensorMap(w, 128)
    pos = torch.arange(200, dtype=torch.int32, device=DEV)
    with pytest.raises(KernelError, match="head sizes"):
        ops.gemm_prompt(x, wm, 6 * 48, torch.empty(200, 4 * 48, dtype=torch.bfloat16, device=DEV), ops.TC_QKV_PREP,
                        prep=dict(nq=4, nkv=1, hd=48, tok_pos=pos))
    with pytest.raises(KernelError, match="writes"):
        ops.gemm_prompt(x, wm, 6 * 48, torch.empty(200, 6 * 48, dtype=torch.float32, device=DEV), ops.TC_STORE_BF16)
    with pytest.raises(KernelError, match="norm-ahead"):
        y = torch.empty(200, 6 * 48, dtype=torch.bfloat16, device=DEV)
        ops.gemm_prompt(x, wm, 6 * 48, y, ops.TC_STORE_BF16,
                        norm_ahead=(torch.ones(6 * 48, device=DEV), torch.empty_like(y), torch.empty(2, 200, device=DEV)))
