"""Each kernel alone against a plain fp32 PyTorch statement of the same operation, at sizes other
than the engine's."""
import math

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def rel(a, b):
    a, b = a.double().flatten(), b.double().flatten()
    return float((a - b).norm() / b.norm().clamp_min(1e-30))


def ref_epilogue(c, epilogue, prev=None):
    if epilogue == 3:
        g, u = c[:, 0::2], c[:, 1::2]
        return g / (1 + torch.exp(-g)) * u
    if epilogue == 2:
        return prev + c
    return c


@pytest.mark.parametrize("M,N,K", [(1, 512, 64), (3, 1000, 96), (17, 192, 200), (64, 2048, 2048), (65, 130, 72),
                                   (128, 256, 512), (129, 1000, 264), (300, 1536, 1024), (1000, 520, 136),
                                   (8, 4096, 2048), (5, 2048, 6144), (16, 12288, 1024), (100, 640, 4096),
                                   (2048, 4096, 512), (777, 1500, 320), (4200, 2300, 136), (130, 100, 64),
                                   (512, 2048, 6144), (260, 204, 1544)])      # few tiles, long K: the adding epilogue cuts K
@pytest.mark.parametrize("epilogue", [0, 1, 2, 3])
@pytest.mark.parametrize("split_mode", [0, 1, 2, 3, 4, 5])
def test_gemm_tc(M, N, K, epilogue, split_mode):
    """split_mode: 0 as the engine chooses, 1 atomics, 2 cluster sums, 3 one tile per block, 4 pairs of SMs
    (tcgen05 cta_group::2) where the shape allows, 5 never pairs."""
    from ember_b200 import ops
    torch.manual_seed(M * 7 + N + K + epilogue)
    a = (torch.randn(M, K, device="cuda") * 0.5).bfloat16()
    w = (torch.randn(N, K, device="cuda") * 0.5).bfloat16()
    n_out = N // 2 if epilogue == 3 else N
    prev = torch.randn(M, n_out, device="cuda")
    out = prev.clone() if epilogue in (1, 2) else torch.zeros(M, n_out, device="cuda", dtype=torch.bfloat16)
    err = torch.zeros(1, dtype=torch.int32, device="cuda")
    assert ops.gemm_tc_usable(a, w, None, epilogue)
    ops.gemm_tc(a, w, out, M, epilogue, err=err, split_mode=split_mode)
    want = ref_epilogue(a.float() @ w.float().t(), epilogue, prev)
    assert int(err.item()) == 0
    tol = 5e-3 if epilogue in (0, 3) else 1e-5          # bf16 rounding of the output, else fp32 accumulation only
    assert rel(out.float(), want) < tol
    if M <= 128:                                        # the split-K scratch is left zeroed
        assert float(ops._tc_scratch[a.device].abs().max()) == 0.0


@pytest.mark.parametrize("M,N,K", [(17, 2048, 264), (64, 2048, 2048), (128, 24576, 128), (100, 640, 264), (33, 1000, 72),
                                   (128, 1160, 136), (70, 20000, 64)])
@pytest.mark.parametrize("epilogue", [0, 1, 3])
def test_gemm_tc_whole_k_more_than_16_tokens(M, N, K, epilogue):
    """17 to 128 tokens with K in one part (forced with split_mode 17, and what the planner picks for a matrix of
    more tiles than SMs): the block turns its tile in shared memory and stores whole pieces of token rows.  1,000
    and 1,160 weight rows end inside a tile (that tile is stored element by element), 1,000 outputs a row are
    no multiple of 16 bytes for the gated epilogue."""
    from ember_b200 import ops
    torch.manual_seed(M + N + K + epilogue)
    a = (torch.randn(M, K, device="cuda") * 0.5).bfloat16()
    w = (torch.randn(N, K, device="cuda") * 0.5).bfloat16()
    n_out = N // 2 if epilogue == 3 else N
    want = ref_epilogue(a.float() @ w.float().t(), epilogue)
    for mode in (17, 0):
        out = torch.full((M + 1, n_out), 7.0, device="cuda", dtype=torch.float32 if epilogue == 1 else torch.bfloat16)
        err = torch.zeros(1, dtype=torch.int32, device="cuda")
        ops.gemm_tc(a, w, out, M, epilogue, err=err, split_mode=mode)
        assert int(err.item()) == 0
        assert rel(out[:M].float(), want) < (5e-3 if epilogue in (0, 3) else 1e-5)
        assert float((out[M].float() - 7.0).abs().max()) == 0.0          # the row after the step's tokens is not touched


@pytest.mark.parametrize("cols", [64, 208, 240])
@pytest.mark.parametrize("split_mode", [4, 5])
def test_gemm_tc_tile_widths(cols, split_mode, monkeypatch):
    """Every tile width the shape heuristic may choose, forced, on one SM and on pairs."""
    from ember_b200 import ops
    monkeypatch.setenv("EMBER_GEMM_TILE_COLS", str(cols))
    torch.manual_seed(cols)
    M, N, K = 700, 1000, 264
    a = (torch.randn(M, K, device="cuda") * 0.5).bfloat16()
    w = (torch.randn(N, K, device="cuda") * 0.5).bfloat16()
    err = torch.zeros(1, dtype=torch.int32, device="cuda")
    for epilogue in (0, 2, 3):
        n_out = N // 2 if epilogue == 3 else N
        prev = torch.randn(M, n_out, device="cuda")
        out = prev.clone() if epilogue == 2 else torch.zeros(M, n_out, device="cuda", dtype=torch.bfloat16)
        ops.gemm_tc(a, w, out, M, epilogue, err=err, split_mode=split_mode)
        want = ref_epilogue(a.float() @ w.float().t(), epilogue, prev)
        assert int(err.item()) == 0
        assert rel(out.float(), want) < (5e-3 if epilogue in (0, 3) else 1e-5)


@pytest.mark.parametrize("M,N,K", [(1, 50, 7), (5, 1000, 96), (70, 130, 33), (200, 192, 64)])
@pytest.mark.parametrize("epilogue", [0, 1, 2, 3])
@pytest.mark.parametrize("adt,wdt", [(torch.float32, torch.float32), (torch.bfloat16, torch.bfloat16),
                                     (torch.bfloat16, torch.float32)])
def test_gemm_simt(M, N, K, epilogue, adt, wdt):
    from ember_b200 import ops
    torch.manual_seed(M + N + K)
    a = (torch.randn(M, K, device="cuda") * 0.5).to(adt)
    w = (torch.randn(N, K, device="cuda") * 0.5).to(wdt)
    bias = torch.randn(N, device="cuda")
    n_out = N // 2 if epilogue == 3 else N
    prev = torch.randn(M, n_out, device="cuda")
    out = prev.clone() if epilogue in (1, 2) else torch.zeros(M, n_out, device="cuda", dtype=adt)
    ops.gemm_simt(a, w, out, M, epilogue, bias=bias)
    c = (a.double() @ w.double().t() + bias.double()).float()
    want = ref_epilogue(c, epilogue, prev)
    tol = 5e-3 if (adt == torch.bfloat16 and epilogue in (0, 3)) else 2e-6
    assert rel(out.float(), want) < tol


def test_gemm_simt_is_independent_of_the_batch():
    """A row's fp32 result is bit-identical whatever else is in the batch."""
    from ember_b200 import ops
    torch.manual_seed(0)
    a = torch.randn(150, 200, device="cuda")
    w = torch.randn(300, 200, device="cuda")
    full = torch.empty(150, 300, device="cuda")
    ops.gemm_simt(a, w, full, 150, 1)
    one = torch.empty(1, 300, device="cuda")
    ops.gemm_simt(a[77:78].contiguous(), w, one, 1, 1)
    assert torch.equal(one[0], full[77])


@pytest.mark.parametrize("H", [64, 96, 1000, 2048, 5120])
@pytest.mark.parametrize("odt", [torch.float32, torch.bfloat16])
def test_rmsnorm(H, odt):
    from ember_b200 import ops
    torch.manual_seed(H)
    x = torch.randn(37, H, device="cuda") * 3
    w = 1 + 0.1 * torch.randn(H, device="cuda")
    rows = torch.tensor([5, 0, 36, 5], dtype=torch.int32, device="cuda")
    for eps in (1e-6, 1e-5):
        out = torch.empty(37, H, device="cuda", dtype=odt)
        ops.rmsnorm(x, w, eps, out, 37)
        want = w * (x * torch.rsqrt((x.double() ** 2).mean(-1, keepdim=True) + eps).float())
        assert rel(out.float(), want) < (4e-3 if odt == torch.bfloat16 else 1e-6)
        g = torch.empty(4, H, device="cuda", dtype=odt)
        ops.rmsnorm(x, w, eps, g, 4, rows=rows)
        assert torch.equal(g, out[rows.long()])


@pytest.mark.parametrize("H", [512, 1024, 2048, 4096, 640])
@pytest.mark.parametrize("odt", [torch.float32, torch.bfloat16])
def test_rmsnorm_many_rows(H, odt):
    """A prompt portion's worth of rows, one of them of another magnitude, and a gathered subset."""
    from ember_b200 import ops
    torch.manual_seed(H + 1)
    n = 1003
    x = torch.randn(n, H, device="cuda") * 3
    x[17] *= 1e3                                               # one row of another magnitude
    w = 1 + 0.1 * torch.randn(H, device="cuda")
    out = torch.full((n + 1, H), 7.0, device="cuda", dtype=odt)
    ops.rmsnorm(x, w, 1e-6, out, n)
    want = w * (x * torch.rsqrt((x.double() ** 2).mean(-1, keepdim=True) + 1e-6).float())
    assert rel(out[:n].float(), want) < (4e-3 if odt == torch.bfloat16 else 1e-6)
    worst = ((out[:n].float() - want).norm(dim=-1) / want.norm(dim=-1)).max()
    assert float(worst) < (6e-3 if odt == torch.bfloat16 else 2e-6)
    assert float((out[n].float() - 7.0).abs().max()) == 0.0    # the row beyond is not touched
    rows = torch.randperm(n, device="cuda")[:300].int()
    g = torch.empty(300, H, device="cuda", dtype=odt)
    ops.rmsnorm(x, w, 1e-6, g, 300, rows=rows)
    assert torch.equal(g, out[rows.long()])


@pytest.mark.parametrize("tdt", [torch.float32, torch.bfloat16])
def test_embed(tdt):
    from ember_b200 import ops
    table = torch.randn(1000, 96, device="cuda").to(tdt)
    toks = torch.tensor([0, 999, 5, 5, 123], dtype=torch.int32, device="cuda")
    out = torch.empty(5, 96, device="cuda")
    err = torch.zeros(1, dtype=torch.int32, device="cuda")
    ops.embed(toks, table, out, err=err)
    assert torch.equal(out, table[toks.long()].float()) and int(err.item()) == 0
    bad = torch.tensor([3, 1000], dtype=torch.int32, device="cuda")
    ops.embed(bad, table, out, err=err)                 # out of range: recorded, not trapped
    assert int(err.item()) == 1 and float(out[1].abs().max()) == 0.0


def rope_ref(x, pos, inv_freq, rotary):
    half = rotary // 2
    ang = pos.float()[:, None] * inv_freq[None, :]
    cs, sn = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    a, b = x[..., :half], x[..., half:rotary]
    return torch.cat([a * cs - b * sn, b * cs + a * sn, x[..., rotary:]], dim=-1)


@pytest.mark.parametrize("heads,kv,D,rotary,page", [(4, 2, 16, 16, 16), (6, 1, 32, 32, 16), (5, 5, 48, 24, 32),
                                                    (16, 8, 128, 128, 16), (3, 1, 256, 256, 64), (2, 2, 80, 0, 16),
                                                    (5, 3, 128, 0, 32), (3, 3, 128, 64, 16)])
@pytest.mark.parametrize("dt", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("norm", [True, False])
def test_qk_norm_rope_store(heads, kv, D, rotary, page, dt, norm):
    from ember_b200 import ops
    torch.manual_seed(heads * D + rotary)
    dev = "cuda"
    lens, starts = [5, 1, 40], [3, 77, 0]                 # three runs at different positions
    T = sum(lens)
    pos = torch.cat([torch.arange(s, s + n) for s, n in zip(starts, lens)]).int().to(dev)
    seq = torch.cat([torch.full((n,), i) for i, n in enumerate(lens)]).int().to(dev)
    nblk = max((s + n + page - 1) // page for s, n in zip(starts, lens))
    pages = 3 * nblk + 2
    perm = torch.randperm(pages)[:3 * nblk].reshape(3, nblk).int().to(dev)      # scattered, out-of-order pages
    ld = (heads + 2 * kv) * D
    qkv = (torch.randn(T, ld, device=dev) * 2).to(dt)
    qw, kw = (1 + 0.1 * torch.randn(D, device=dev), 1 + 0.1 * torch.randn(D, device=dev)) if norm else (None, None)
    inv = (1.0 / (10000.0 ** (torch.arange(rotary // 2, device=dev).float() * 2 / max(rotary, 1)))) if rotary else None
    kp = torch.zeros(pages, kv, page, D, device=dev, dtype=dt)
    vp = torch.zeros_like(kp)
    q = torch.empty(T, heads * D, device=dev, dtype=dt)
    err = torch.zeros(1, dtype=torch.int32, device=dev)
    ops.qk_norm_rope_store(qkv, T, heads, kv, D, qw, kw, 1e-5, inv, rotary, pos, seq, perm, page, kp, vp, q, err=err)
    assert int(err.item()) == 0
    x = qkv.float()
    qq, kk, vv = x[:, :heads * D].view(T, heads, D), x[:, heads * D:(heads + kv) * D].view(T, kv, D), x[:, (heads + kv) * D:].view(T, kv, D)

    def nrm(t, w):
        return w * (t * torch.rsqrt((t.double() ** 2).mean(-1, keepdim=True) + 1e-5).float()) if norm else t

    qq, kk = nrm(qq, qw), nrm(kk, kw)
    if rotary:
        qq, kk = rope_ref(qq, pos, inv, rotary), rope_ref(kk, pos, inv, rotary)
    tol = 6e-3 if dt == torch.bfloat16 else 2e-6
    assert rel(q.float().view(T, heads, D), qq) < tol
    for t in range(T):
        blk, slot = int(perm[seq[t], pos[t] // page]), int(pos[t]) % page
        assert rel(kp[blk, :, slot].float(), kk[t]) < tol
        assert torch.equal(vp[blk, :, slot].float(), vv[t].to(dt).float())
    written = torch.zeros(pages, page, dtype=torch.bool)
    for t in range(T):
        written[int(perm[seq[t], pos[t] // page]), int(pos[t]) % page] = True
    untouched = kp.permute(0, 2, 1, 3)[~written.to(dev)]
    assert float(untouched.abs().max() if untouched.numel() else 0) == 0.0             # nothing else was touched


def attention_ref(q, k, v, scale, window):
    T, H, D = q.shape
    G = H // k.shape[1]
    out = torch.zeros_like(q)
    n = k.shape[0]
    for h in range(H):
        s = (q[:, h] @ k[:, h // G].t()) * scale
        qpos = torch.arange(n - T, n, device=q.device)[:, None]
        kpos = torch.arange(n, device=q.device)[None, :]
        vis = kpos <= qpos
        if window:
            vis &= kpos > qpos - window
        out[:, h] = torch.softmax(s.masked_fill(~vis, float("-inf")), -1) @ v[:, h // G]
    return out


@pytest.mark.parametrize("heads,kv,D,page", [(4, 2, 16, 16), (6, 1, 32, 16), (8, 8, 64, 32), (16, 8, 128, 16), (2, 1, 256, 16),
                                             (12, 4, 80, 16), (12, 2, 128, 64), (5, 1, 64, 16), (32, 2, 64, 16),
                                             (8, 8, 128, 32), (8, 2, 128, 16), (16, 1, 128, 16)])
@pytest.mark.parametrize("dt", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("window", [0, 37])
def test_attention_general(heads, kv, D, page, dt, window):
    """Runs of different lengths at different cache depths, scattered pages, one far key made to
    stand out so that a wrong page or a wrong mask shows."""
    from ember_b200 import ops
    from ember_b200.engine.batch import StepBatch, attention_tiles
    torch.manual_seed(heads + D + window)
    dev = "cuda"
    ctx_lens, new = [300, 45, 1, 700], [33, 45, 1, 1]       # tokens cached after the step, new tokens of it
    S = len(ctx_lens)
    nblk = max((c + page - 1) // page for c in ctx_lens)
    pages = S * nblk + 3
    perm = torch.randperm(pages)[:S * nblk].reshape(S, nblk).int()
    kp = torch.zeros(pages, kv, page, D, dtype=dt)
    vp = torch.zeros_like(kp)
    ks, vs, qs = [], [], []
    for s in range(S):
        k = torch.randn(ctx_lens[s], kv, D) * 0.5
        v = torch.randn(ctx_lens[s], kv, D)
        q = torch.randn(new[s], heads, D) * 0.5
        if ctx_lens[s] > 100:                               # one far key stands out for the last query
            far = 7 if not window else ctx_lens[s] - window + 1
            k[far] = q[-1, ::heads // kv] * 6.0
        ks.append(k.to(dt).float()), vs.append(v.to(dt).float()), qs.append(q.to(dt).float())
        for j in range(ctx_lens[s]):
            kp[perm[s, j // page], :, j % page] = k[j].to(dt)
            vp[perm[s, j // page], :, j % page] = v[j].to(dt)
    T = sum(new)
    q_all = torch.cat(qs).to(dt).to(dev).contiguous()
    qstart = np.cumsum([0] + new).astype(np.int32)
    positions = np.concatenate([np.arange(c - n, c) for c, n in zip(ctx_lens, new)]).astype(np.int32)
    batch = StepBatch(requests=list(range(S)), tokens=np.zeros(T, np.int32), positions=positions,
                      seq_of=np.repeat(np.arange(S), new).astype(np.int32), query_start=qstart,
                      context_len=np.asarray(ctx_lens, np.int32), block_tables=[perm.numpy()],
                      state_slots=np.zeros(S, np.int32), logit_rows=np.zeros(0, np.int32))
    tile_q = ops.attention_tile_queries(heads // kv)
    tiles = torch.from_numpy(attention_tiles(batch, tile_q)).to(dev)
    scale = 1.0 / math.sqrt(D)
    want = torch.cat([attention_ref(qs[s].to(dev), ks[s].to(dev), vs[s].to(dev), scale, window) for s in range(S)])
    err = torch.zeros(1, dtype=torch.int32, device=dev)
    if dt == torch.bfloat16 and ops.attention_tc_supported(D, heads // kv, page, 0):
        # the tensor-core kernels on the same case: prompt portions in mode 0, single tokens in mode 1
        out = torch.zeros(T, heads * D, device=dev, dtype=dt)
        tq = ops.attention_tc_tile_queries(heads // kv)
        multi = torch.from_numpy(attention_tiles(batch, tq, "multi")).to(dev)
        single = torch.from_numpy(attention_tiles(batch, 1, "single")).to(dev)
        ops.attention_tc(q_all.view(T, -1), kp.to(dev), vp.to(dev), out, 0, heads, kv, D, multi, multi.shape[0],
                         perm.to(dev), page, window, scale, err=err)
        # splits merged by a second kernel through buffers, or (no buffers, at most 8) inside a cluster
        for n_splits, split_keys, buffers in ((1, 0, True), (4, 192, True), (11, 64, True), (4, 192, False), (8, 128, False),
                                              (3, 320, False)):
            po = torch.empty(single.shape[0] * heads * n_splits * D, device=dev) if buffers else None
            pml = torch.empty(single.shape[0] * heads * n_splits * 2, device=dev) if buffers else None
            out[-2:] = 0
            ops.attention_tc(q_all.view(T, -1), kp.to(dev), vp.to(dev), out, 1, heads, kv, D, single, single.shape[0],
                             perm.to(dev), page, window, scale, n_splits, split_keys, po, pml, err=err)
            assert int(err.item()) == 0
            assert rel(out.float().view(T, heads, D), want) < 6e-3
        all_tiles = torch.from_numpy(attention_tiles(batch, tq, "all")).to(dev)     # single tokens through mode 0 too
        out2 = torch.zeros_like(out)
        ops.attention_tc(q_all.view(T, -1), kp.to(dev), vp.to(dev), out2, 0, heads, kv, D, all_tiles, all_tiles.shape[0],
                         perm.to(dev), page, window, scale, err=err)
        assert int(err.item()) == 0 and rel(out2.float().view(T, heads, D), want) < 6e-3
    if dt == torch.bfloat16 and ops.attention_fa_supported(D, heads // kv, page):
        # the tcgen05 kernel on the prompt portions of the same case
        out = torch.zeros(T, heads * D, device=dev, dtype=dt)
        tq = ops.attention_fa_tile_queries(heads // kv)
        multi = torch.from_numpy(attention_tiles(batch, tq, "multi")).to(dev)
        ops.attention_fa(q_all.view(T, -1), kp.to(dev), vp.to(dev), out, heads, kv, D, multi, multi.shape[0],
                         perm.to(dev), page, window, scale, err=err)
        assert int(err.item()) == 0
        n_multi = sum(n for n in new if n > 1)
        assert rel(out.float().view(T, heads, D)[:n_multi], want[:n_multi]) < 6e-3
    for n_splits, split_keys in ((1, 0), (6, 128)):
        out = torch.zeros(T, heads * D, device=dev, dtype=dt)
        po = torch.empty(T * heads * n_splits * D, device=dev)
        pml = torch.empty(T * heads * n_splits * 2, device=dev)
        ops.attention(q_all.view(T, -1), kp.to(dev), vp.to(dev), out, T, heads, kv, D, tiles, tiles.shape[0], tile_q,
                      perm.to(dev), page, window, scale, n_splits, split_keys, po, pml, err=err)
        assert int(err.item()) == 0
        assert rel(out.float().view(T, heads, D), want) < (6e-3 if dt == torch.bfloat16 else 3e-6)


@pytest.mark.parametrize("page", [16, 64])
def test_attention_long_context(page):
    """Contexts beyond 8,192 keys at the benchmark's head geometry: a 2,048-token portion whose first query already
    sees 8,200 cached keys (the tcgen05 kernel), and single tokens over 9,000 and 12,345 keys with the key range cut
    into 16 splits, the most the planner makes, and into one (the TMA-fed decode kernel).  For the last query of
    every run one key in the second page is made to stand out, for the first query of the portion the key just
    before it, so that a far page that is skipped, fetched twice or merged with the wrong weight shows."""
    from ember_b200 import ops
    from ember_b200.engine.batch import StepBatch, attention_tiles
    heads, kv, D, dt, dev = 16, 8, 128, torch.bfloat16, "cuda"
    torch.manual_seed(page)
    ctx_lens, new = [8200 + 2048, 9000, 12345], [2048, 1, 1]
    S = len(ctx_lens)
    nblk = max((c + page - 1) // page for c in ctx_lens)
    pages = S * nblk + 5
    perm = torch.randperm(pages)[:S * nblk].reshape(S, nblk).int()
    kp = torch.zeros(pages, kv, page, D, dtype=dt)
    vp = torch.zeros_like(kp)
    ks, vs, qs = [], [], []
    for s in range(S):
        k = torch.randn(ctx_lens[s], kv, D) * 0.5
        v = torch.randn(ctx_lens[s], kv, D)
        q = torch.randn(new[s], heads, D) * 0.5
        k[page + 3] = q[-1, ::heads // kv] * 4.0
        if new[s] > 1:
            k[ctx_lens[s] - new[s] - 1] = q[0, ::heads // kv] * 4.0
        ks.append(k.to(dt).float()), vs.append(v.to(dt).float()), qs.append(q.to(dt).float())
        for b in range(nblk):
            lo, hi = b * page, min((b + 1) * page, ctx_lens[s])
            if lo < hi:
                kp[perm[s, b], :, :hi - lo] = k[lo:hi].to(dt).transpose(0, 1)
                vp[perm[s, b], :, :hi - lo] = v[lo:hi].to(dt).transpose(0, 1)
    T = sum(new)
    q_all = torch.cat(qs).to(dt).to(dev).contiguous()
    positions = np.concatenate([np.arange(c - n, c) for c, n in zip(ctx_lens, new)]).astype(np.int32)
    batch = StepBatch(requests=list(range(S)), tokens=np.zeros(T, np.int32), positions=positions,
                      seq_of=np.repeat(np.arange(S), new).astype(np.int32), query_start=np.cumsum([0] + new).astype(np.int32),
                      context_len=np.asarray(ctx_lens, np.int32), block_tables=[perm.numpy()],
                      state_slots=np.zeros(S, np.int32), logit_rows=np.zeros(0, np.int32))
    scale = 1.0 / math.sqrt(D)
    want = torch.cat([attention_ref(qs[s].to(dev), ks[s].to(dev), vs[s].to(dev), scale, 0) for s in range(S)])
    err = torch.zeros(1, dtype=torch.int32, device=dev)
    kd, vd, pd = kp.to(dev), vp.to(dev), perm.to(dev)
    out = torch.zeros(T, heads * D, device=dev, dtype=dt)
    multi = torch.from_numpy(attention_tiles(batch, ops.attention_fa_tile_queries(heads // kv), "multi")).to(dev)
    ops.attention_fa(q_all.view(T, -1), kd, vd, out, heads, kv, D, multi, multi.shape[0], pd, page, 0, scale, err=err)
    single = torch.from_numpy(attention_tiles(batch, 1, "single")).to(dev)
    longest = max(ctx_lens)
    for n_splits, buffers in ((16, True), (1, True), (8, False), (5, False)):
        split_keys = ((longest + n_splits - 1) // n_splits + 63) // 64 * 64 if n_splits > 1 else 0
        po = torch.empty(single.shape[0] * heads * n_splits * D, device=dev) if buffers else None
        pml = torch.empty(single.shape[0] * heads * n_splits * 2, device=dev) if buffers else None
        out[-2:] = 0
        ops.attention_tc(q_all.view(T, -1), kd, vd, out, 1, heads, kv, D, single, single.shape[0], pd, page, 0, scale,
                         n_splits, split_keys, po, pml, err=err)
        assert int(err.item()) == 0
        rows = (out.float().view(T, heads, D) - want).norm(dim=-1) / want.norm(dim=-1)
        assert float(rows.max()) < 2e-2, (n_splits, float(rows.max()), int(rows.max(dim=-1).values.argmax()))
        assert rel(out.float().view(T, heads, D), want) < 6e-3


@pytest.mark.parametrize("heads,kv,page", [(16, 8, 16), (8, 1, 32), (3, 3, 64)])
@pytest.mark.parametrize("window", [0, 700])
def test_attention_fa_many_blocks(heads, kv, page, window):
    """Long prompt portions: more blocks than the device has SMs, so that blocks share an SM and start
    after others have ended, and short and long key ranges run side by side.  One far key is made to
    dominate the last query of each run, one near key the first, so that a key tile that is lost or
    masked wrongly shows; the launch is repeated because such faults depend on timing."""
    from ember_b200 import ops
    from ember_b200.engine.batch import StepBatch, attention_tiles
    D, dt, dev = 128, torch.bfloat16, "cuda"
    if not ops.attention_fa_supported(D, heads // kv, page):
        pytest.skip("geometry not taken by the tcgen05 kernel")
    torch.manual_seed(heads * page + window)
    ctx_lens, new = [1500, 530, 90, 1100], [700, 200, 90, 600]
    S = len(ctx_lens)
    nblk = max((c + page - 1) // page for c in ctx_lens)
    pages = S * nblk + 3
    perm = torch.randperm(pages)[:S * nblk].reshape(S, nblk).int()
    kp = torch.zeros(pages, kv, page, D, dtype=dt)
    vp = torch.zeros_like(kp)
    ks, vs, qs = [], [], []
    for s in range(S):
        k = torch.randn(ctx_lens[s], kv, D) * 0.5
        v = torch.randn(ctx_lens[s], kv, D)
        q = torch.randn(new[s], heads, D) * 0.5
        far = 5 if not window else max(0, ctx_lens[s] - window + 1)
        k[far] = q[-1, ::heads // kv] * 4.0
        k[ctx_lens[s] - new[s]] = q[0, ::heads // kv] * 4.0
        ks.append(k.to(dt).float()), vs.append(v.to(dt).float()), qs.append(q.to(dt).float())
        for b in range(nblk):
            lo, hi = b * page, min((b + 1) * page, ctx_lens[s])
            if lo < hi:
                kp[perm[s, b], :, :hi - lo] = k[lo:hi].to(dt).transpose(0, 1)
                vp[perm[s, b], :, :hi - lo] = v[lo:hi].to(dt).transpose(0, 1)
    T = sum(new)
    q_all = torch.cat(qs).to(dt).to(dev).contiguous()
    qstart = np.cumsum([0] + new).astype(np.int32)
    positions = np.concatenate([np.arange(c - n, c) for c, n in zip(ctx_lens, new)]).astype(np.int32)
    batch = StepBatch(requests=list(range(S)), tokens=np.zeros(T, np.int32), positions=positions,
                      seq_of=np.repeat(np.arange(S), new).astype(np.int32), query_start=qstart,
                      context_len=np.asarray(ctx_lens, np.int32), block_tables=[perm.numpy()],
                      state_slots=np.zeros(S, np.int32), logit_rows=np.zeros(0, np.int32))
    scale = 1.0 / math.sqrt(D)
    want = torch.cat([attention_ref(qs[s].to(dev), ks[s].to(dev), vs[s].to(dev), scale, window) for s in range(S)])
    tq = ops.attention_fa_tile_queries(heads // kv)
    tiles = torch.from_numpy(attention_tiles(batch, tq, "multi")).to(dev)
    err = torch.zeros(1, dtype=torch.int32, device=dev)
    kd, vd, pd = kp.to(dev), vp.to(dev), perm.to(dev)
    for _ in range(4):
        out = torch.zeros(T, heads * D, device=dev, dtype=dt)
        ops.attention_fa(q_all.view(T, -1), kd, vd, out, heads, kv, D, tiles, tiles.shape[0], pd, page, window, scale, err=err)
        assert int(err.item()) == 0
        worst = ((out.float().view(T, heads, D) - want).norm(dim=-1) / want.norm(dim=-1)).max()
        assert float(worst) < 2e-2                           # every row, not only the sum over rows
        assert rel(out.float().view(T, heads, D), want) < 6e-3


@pytest.mark.parametrize("heads,kv,page,M", [(4, 2, 16, 300), (3, 1, 64, 200), (6, 2, 32, 2100), (5, 1, 16, 2304),
                                             (16, 8, 16, 8), (4, 2, 64, 1), (3, 1, 32, 16), (40, 8, 16, 5)])
@pytest.mark.parametrize("norm,rotate", [(True, True), (False, True), (True, False)])
def test_gemm_tc_qkv(heads, kv, page, M, norm, rotate):
    """The fused q/k/v product: heads finished in the epilogue (norm, rotation, cache write) against the same
    steps computed plainly from the fp32 product.  Two runs at different depths, scattered pages; 2,100 and
    2,304 tokens go to the kernel on pairs of SMs, the others to the single-SM kernel; 3 and 5 + 2 head slots
    give tiles of one head, the others of two."""
    from ember_b200 import ops
    torch.manual_seed(heads * M + page)
    dev, D = "cuda", 128
    K = 136 if M == 5 else 328                         # no multiples of 64; 136: too short to split over a cluster
    lens = [M - 130, 130] if M > 130 else [M - M // 2, M // 2]      # 1..16 tokens: the decode-sized kernel
    starts = [37, 1000]
    pos = torch.cat([torch.arange(s, s + n) for s, n in zip(starts, lens)]).int().to(dev)
    seq = torch.cat([torch.full((n,), i) for i, n in enumerate(lens)]).int().to(dev)
    nblk = max((s + n + page - 1) // page for s, n in zip(starts, lens))
    pages = 2 * nblk + 2
    perm = torch.randperm(pages)[:2 * nblk].reshape(2, nblk).int().to(dev)
    N = (heads + 2 * kv) * D
    a = (torch.randn(M, K, device=dev) * 0.5).bfloat16()
    w = (torch.randn(N, K, device=dev) * 0.1).bfloat16()
    qw, kw = (1 + 0.1 * torch.randn(D, device=dev), 1 + 0.1 * torch.randn(D, device=dev)) if norm else (None, None)
    inv = 1.0 / (10000.0 ** (torch.arange(D // 2, device=dev).float() * 2 / D))
    assert ops.gemm_tc_qkv_usable(a, w, None, M, heads, kv, D, D if rotate else 0)
    cs = None
    if rotate and M <= 16:
        fr = inv
    elif rotate:
        fr = None
        cs = torch.empty(D // 4, M + 8, 4, device=dev)          # rows longer than the step
        ops.rope_table(pos, inv, M, cs)
        ang = pos.float()[None, :] * inv[:, None]                # [frequency, token]
        got = cs[:, :M].view(D // 4, M, 2, 2).permute(0, 3, 1, 2).reshape(D // 2, M, 2)      # (cos, cos, sin, sin) per pair
        assert torch.allclose(got[..., 0], torch.cos(ang), atol=2e-6) and torch.allclose(got[..., 1], torch.sin(ang), atol=2e-6)
    if not rotate:
        fr = None
    x = a.float() @ w.float().t()
    qq, kk, vv = x[:, :heads * D].view(M, heads, D), x[:, heads * D:(heads + kv) * D].view(M, kv, D), x[:, (heads + kv) * D:].view(M, kv, D)

    def nrm(t, g):
        return g * (t * torch.rsqrt((t.double() ** 2).mean(-1, keepdim=True) + 1e-5).float()) if norm else t

    qq, kk = nrm(qq, qw), nrm(kk, kw)
    if rotate:
        qq, kk = rope_ref(qq, pos, inv, D), rope_ref(kk, pos, inv, D)
    for write_kv in (True, False):
        kp = torch.zeros(pages, kv, page, D, device=dev, dtype=torch.bfloat16)
        vp = torch.zeros_like(kp)
        q = torch.zeros(M, heads * D, device=dev, dtype=torch.bfloat16)
        err = torch.zeros(1, dtype=torch.int32, device=dev)
        ops.gemm_tc_qkv(a, w, M, heads, kv, qw, kw, 1e-5, cs, fr, pos, seq, perm, page, kp, vp, q, write_kv=write_kv, err=err)
        assert int(err.item()) == 0
        assert rel(q.float().view(M, heads, D), qq) < 5e-3
        worst = ((q.float().view(M, heads, D) - qq).norm(dim=-1) / qq.norm(dim=-1)).max()
        assert float(worst) < 1.5e-2                          # every head of every token
        if not write_kv:
            assert float(kp.abs().max()) == 0.0 and float(vp.abs().max()) == 0.0
            continue
        blk = perm[seq.long(), (pos // page).long()].long()
        slot = (pos % page).long()
        assert rel(kp[blk, :, slot].float(), kk) < 5e-3
        assert rel(vp[blk, :, slot].float(), vv) < 5e-3
        written = torch.zeros(pages, page, dtype=torch.bool, device=dev)
        written[blk, slot] = True
        untouched = kp.permute(0, 2, 1, 3)[~written]
        assert float(untouched.abs().max() if untouched.numel() else 0) == 0.0
    # a page id outside the pool is recorded, not written
    bad = perm.clone()
    bad[0, starts[0] // page] = pages + 5
    err = torch.zeros(1, dtype=torch.int32, device=dev)
    ops.gemm_tc_qkv(a, w, M, heads, kv, qw, kw, 1e-5, cs, fr, pos, seq, bad, page, kp, vp, q, err=err)
    assert int(err.item()) == 2


@pytest.mark.parametrize("heads,kv,page,M,K", [(16, 8, 64, 64, 2048), (4, 2, 16, 17, 328), (3, 1, 32, 128, 136), (40, 8, 16, 100, 512),
                                               (32, 8, 64, 33, 4096)])
@pytest.mark.parametrize("norm,rotate", [(True, True), (False, True), (True, False)])
def test_qkv_sums_to_heads(heads, kv, page, M, K, norm, rotate):
    """17 to 128 tokens: the q/k/v product leaves its fp32 sums in the scratch (K cut into parts added with atomics,
    or one part stored), the head kernel reads them there, norms, rotates, writes queries and cache, and sets every
    sum back to zero."""
    from ember_b200 import ops
    torch.manual_seed(heads * M + page + K)
    dev, D = "cuda", 128
    lens = [M - M // 3, M // 3]
    starts = [5, 700]
    pos = torch.cat([torch.arange(s, s + n) for s, n in zip(starts, lens)]).int().to(dev)
    seq = torch.cat([torch.full((n,), i) for i, n in enumerate(lens)]).int().to(dev)
    nblk = max((s + n + page - 1) // page for s, n in zip(starts, lens))
    pages = 2 * nblk + 2
    perm = torch.randperm(pages)[:2 * nblk].reshape(2, nblk).int().to(dev)
    N = (heads + 2 * kv) * D
    a = (torch.randn(M, K, device=dev) * 0.5).bfloat16()
    w = (torch.randn(N, K, device=dev) * 0.1).bfloat16()
    qw, kw = (1 + 0.1 * torch.randn(D, device=dev), 1 + 0.1 * torch.randn(D, device=dev)) if norm else (None, None)
    inv = 1.0 / (10000.0 ** (torch.arange(D // 2, device=dev).float() * 2 / D))
    x = a.float() @ w.float().t()
    qq, kk, vv = x[:, :heads * D].view(M, heads, D), x[:, heads * D:(heads + kv) * D].view(M, kv, D), x[:, (heads + kv) * D:].view(M, kv, D)

    def nrm(t, g):
        return g * (t * torch.rsqrt((t.double() ** 2).mean(-1, keepdim=True) + 1e-5).float()) if norm else t

    qq, kk = nrm(qq, qw), nrm(kk, kw)
    if rotate:
        qq, kk = rope_ref(qq, pos, inv, D), rope_ref(kk, pos, inv, D)
    assert ops.qk_norm_rope_store_sums_usable(D, D if rotate else 0, N)
    for write_kv in (True, False):
        kp = torch.zeros(pages, kv, page, D, device=dev, dtype=torch.bfloat16)
        vp = torch.zeros_like(kp)
        q = torch.zeros(M, heads * D, device=dev, dtype=torch.bfloat16)
        err = torch.zeros(1, dtype=torch.int32, device=dev)
        sums = ops.gemm_tc(a, w, None, M, ops.EPI_SUMS, err=err)
        assert rel(sums, x) < 1e-5                       # fp32 sums of the bf16 operands
        ops.qk_norm_rope_store_sums(sums, M, heads, kv, qw, kw, 1e-5, inv if rotate else None, pos, seq, perm, page, kp, vp, q,
                                    write_kv=write_kv, err=err)
        assert int(err.item()) == 0
        assert float(ops._tc_scratch[a.device].abs().max()) == 0.0        # every sum was set back to zero
        assert rel(q.float().view(M, heads, D), qq) < 5e-3
        if not write_kv:
            assert float(kp.abs().max()) == 0.0 and float(vp.abs().max()) == 0.0
            continue
        blk = perm[seq.long(), (pos // page).long()].long()
        slot = (pos % page).long()
        assert rel(kp[blk, :, slot].float(), kk) < 5e-3
        assert rel(vp[blk, :, slot].float(), vv) < 5e-3


def test_bounded_wait_runs_out_and_returns():
    """The wait every TMA / tcgen05 kernel uses, on a barrier nobody arrives at, with a limit of one millisecond:
    the kernel returns, the error word holds the wait-limit bit, the wait lasted about the limit (not a poll
    count's worth of unknown time), the runner turns the word into a DeviceError, and the device works afterwards."""
    from ember_b200 import ops
    from ember_b200.engine.runner import ModelRunner
    dev = "cuda"
    err = torch.zeros(1, dtype=torch.int32, device=dev)
    waited = torch.zeros(1, dtype=torch.int64, device=dev)
    ops.wait_limit_probe(1_000_000, err, waited)
    torch.cuda.synchronize()
    assert int(err.item()) == 4                                   # EMBER_ERR_WAIT_LIMIT
    assert 1_000_000 <= int(waited.item()) < 50_000_000
    assert "a bounded wait ran out" in ModelRunner.describe_error(int(err.item()))
    with pytest.raises(ops.KernelError):
        ops.wait_limit_probe(10_000_000_000, err, waited)          # a limit a test should not ask for
    x = torch.randn(4, 64, device=dev)
    out = torch.empty(4, 64, device=dev)
    ops.rmsnorm(x, torch.ones(64, device=dev), 1e-6, out, 4)
    assert torch.isfinite(out).all()
