"""Each kernel alone against a plain PyTorch FP32 reference of the same operation, at sizes other
than the engine's tiny configurations (odd widths, head sizes in steps of 16, ragged groups)."""
import math

import pytest
import torch

import helpers
import plain_flint as P

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _t(*shape, dtype=torch.float32, scale=1.0, seed=0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(*shape, generator=g) * scale).to(dtype).to(DEV)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("V,D,T", [(50, 24, 7), (333, 100, 19)])
def test_embed(dtype, V, D, T):
    from quench6k_b200 import ops
    table = _t(V, D, dtype=dtype)
    tok = torch.randint(0, V, (T,), dtype=torch.int32, device=DEV)
    out = ops.embed(tok, table)
    assert torch.equal(out, table[tok.long()].float())


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("R,D,eps", [(5, 72, 1e-6), (33, 2048, 1e-5), (3, 1000, 1e-3)])
def test_rmsnorm(dtype, R, D, eps):
    from quench6k_b200 import ops
    x, w = _t(R, D, scale=3.0), _t(D, seed=1) + 1.0
    out = ops.rmsnorm(x, w, eps, dtype)
    ref = P.rmsnorm(x.double().cpu(), w.double().cpu(), eps)
    tol = 1e-5 if dtype == torch.float32 else 1e-2
    assert (out.double().cpu() - ref).abs().max() <= tol * ref.abs().max()
    rows = torch.tensor([R - 1, 0, 2], dtype=torch.int32, device=DEV)
    sel = ops.rmsnorm(x, w, eps, dtype, rows=rows)
    assert torch.equal(sel, out[rows.long()])
    add = _t(R, D, seed=3)
    x2 = x.clone()
    fused = ops.rmsnorm(x2, w, eps, dtype, add=add)
    assert torch.equal(x2, x + add)
    assert torch.equal(fused, ops.rmsnorm(x + add, w, eps, dtype))
    # the routed experts' results added inside the norm: the same values as combine followed by the norm
    S = 3
    y, sw = _t(R * S + 2, D, seed=4), _t(R, S, seed=5)
    perm = torch.randperm(R * S, generator=torch.Generator().manual_seed(6)).to(torch.int32).view(R, S).to(DEV)
    for pair_row in (None, perm):
        for sel in (None, rows):
            xa, xb = x.clone(), x.clone()
            ops.combine(y, pair_row, sw, xa)
            want = ops.rmsnorm(xa, w, eps, dtype, rows=sel)
            got = ops.rmsnorm(xb, w, eps, dtype, rows=sel, weighted=(y, pair_row, sw))
            assert torch.equal(got, want)
            touched = torch.arange(R, device=DEV) if sel is None else sel.long()
            assert torch.equal(xb[touched], xa[touched])


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("M,N,K", [(1, 70, 33), (65, 129, 100), (200, 64, 257), (3, 1000, 72)])
def test_gemm_simt(dtype, M, N, K):
    from quench6k_b200 import ops
    a, w = _t(M, K, dtype=dtype), _t(N, K, dtype=dtype, seed=1)
    ref = a.double().cpu() @ w.double().cpu().T
    out = ops.gemm_simt(a, w)
    assert out.dtype == torch.float32
    assert (out.double().cpu() - ref).abs().max() <= 2e-5 * math.sqrt(K) * ref.abs().max()
    base = _t(M, N, seed=2)
    acc = base.clone()
    ops.gemm_simt(a, w, out=acc, accumulate=True)
    assert (acc.double().cpu() - (base.double().cpu() + ref)).abs().max() <= 2e-5 * math.sqrt(K) * ref.abs().max()
    # rows do not depend on the batch they are in
    one = ops.gemm_simt(a[M // 2:M // 2 + 1].contiguous(), w)
    assert torch.equal(one[0], out[M // 2])
    w2 = _t(N, K, dtype=dtype, seed=3)
    act = ops.gemm_simt(a, w, w2=w2)
    g, u = ref, a.double().cpu() @ w2.double().cpu().T
    want = P.silu(g) * u
    tol = 1e-5 if dtype == torch.float32 else 1e-2
    assert act.dtype == dtype
    assert (act.double().cpu() - want).abs().max() <= tol * math.sqrt(K) * want.abs().max()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_grouped_gemm_and_permutation(dtype):
    from quench6k_b200 import ops
    T, k, E, D, I = 37, 3, 10, 56, 24
    g = torch.Generator().manual_seed(4)
    sel = torch.stack([torch.randperm(E, generator=g)[:k] for _ in range(T)]).to(torch.int32).to(DEV)
    sel[:, 0] = torch.where(sel[:, 0] == 7, sel[:, 1], sel[:, 0])         # leave expert 7 nearly empty
    offsets, pair_row, row_token = ops.moe_permute(sel, E)
    flat = sel.flatten().cpu()
    order = torch.sort(flat, stable=True).indices
    assert offsets.cpu().tolist() == [int((flat < e).sum()) for e in range(E + 1)]
    assert torch.equal(row_token.cpu().long(), order // k)
    assert torch.equal(pair_row.flatten().cpu().long()[order], torch.arange(T * k))
    groups = ops.tile_list(offsets, T * k, ops.simt_tile_rows())
    x, wg, wu = _t(T, D, dtype=dtype), _t(E, I, D, dtype=dtype, seed=1), _t(E, I, D, dtype=dtype, seed=2)
    wd = _t(E, D, I, dtype=dtype, seed=3)
    act = ops.gemm_simt(x, wg, w2=wu, a_rows=row_token, groups=groups, rows=T * k)
    y = ops.gemm_simt(act, wd, groups=groups, rows=T * k)
    tol = 1e-5 if dtype == torch.float32 else 2e-2
    for row in range(T * k):
        e, t = int(flat[order[row]]), int(order[row]) // k
        xa = x[t].double().cpu()
        a_ref = P.silu(wg[e].double().cpu() @ xa) * (wu[e].double().cpu() @ xa)
        assert (act[row].double().cpu() - a_ref).abs().max() <= tol * a_ref.abs().max() + 1e-9
        y_ref = wd[e].double().cpu() @ act[row].double().cpu()
        assert (y[row].double().cpu() - y_ref).abs().max() <= 1e-4 * y_ref.abs().max() + 1e-9
    w = torch.rand(T, k, generator=g).to(DEV)
    h = _t(T, D, seed=9)
    want = h.double().cpu() + (w.double().cpu()[:, :, None] * y.double().cpu()[pair_row.cpu().long()]).sum(1)
    ops.combine(y, pair_row, w, h)
    assert (h.double().cpu() - want).abs().max() <= 1e-5 * want.abs().max()


@pytest.mark.parametrize("T,k,E,D,bm", [(37, 3, 10, 56, 16), (2048, 8, 256, 64, 128), (300, 1, 7, 8, 32), (1500, 6, 33, 24, 64),
                                        (700, 4, 1024, 16, 32), (515, 5, 1500, 40, 16)])
def test_moe_plan_equals_its_parts(T, k, E, D, bm):
    """Permutation and tile list in three launches against the four single ones: the same arrays."""
    from quench6k_b200 import ops
    g = torch.Generator().manual_seed(T + E)
    sel = torch.stack([torch.randperm(E, generator=g)[:k] for _ in range(T)]).to(torch.int32).to(DEV)
    offsets, pair_row, row_token = ops.moe_permute(sel, E)
    tiles = ops.tile_list(offsets, T * k, bm)
    o2, p2, r2, t2 = ops.moe_plan(sel, E, bm)
    assert torch.equal(o2, offsets) and torch.equal(p2, pair_row) and torch.equal(r2, row_token)
    n = int(tiles[3])
    assert int(t2[3]) == n and torch.equal(t2[1][:n], tiles[1][:n]) and torch.equal(t2[2][:n], tiles[2][:n])
    # with the pairs' input rows copied into place by the last launch
    x = _t(T, D, dtype=torch.bfloat16, seed=3)
    o3, p3, r3, t3, xs = ops.moe_plan(sel, E, bm, x)
    assert torch.equal(o3, offsets) and torch.equal(p3, pair_row) and torch.equal(r3, row_token) and int(t3[3]) == n
    assert torch.equal(xs, x[row_token.long()])


@pytest.mark.parametrize("scoring", ["softmax", "sigmoid"])
@pytest.mark.parametrize("renorm", [True, False])
@pytest.mark.parametrize("T,E,k", [(9, 6, 3), (40, 256, 8), (5, 100, 100), (7, 500, 9), (3, 3000, 6), (2, 1500, 40)])
def test_route(scoring, renorm, T, E, k):
    from quench6k_b200 import ops
    z = _t(T, E, scale=2.0)
    z[:, 1] = z[:, 0]                                                    # ties
    z = (z * 4).round() / 4
    sel, w = ops.route(z, k, scoring, renorm)
    rsel, rw = P.route(z.cpu().float(), scoring, k, renorm)
    assert torch.equal(sel.cpu().long(), rsel)
    assert (w.cpu() - rw).abs().max() <= 1e-5 * rw.abs().max()
    # the same logits as three split-K slices (quarters of the values, which add up exactly)
    parts = torch.stack([z / 2, z / 4, z / 4]).contiguous()
    sel3, w3 = ops.route(parts, k, scoring, renorm)
    assert torch.equal(sel3, sel) and torch.equal(w3, w)


def _paged(k, v, page_size, num_pages, dtype, seed):
    """Scatter whole-sequence k, v [T, Hkv, hd] into randomly chosen pages; returns pages and the table."""
    T, Hkv, hd = k.shape
    nb = (T + page_size - 1) // page_size
    g = torch.Generator().manual_seed(seed)
    table = torch.randperm(num_pages, generator=g)[:nb].to(torch.int32)
    kp = torch.full((Hkv, num_pages, page_size, hd), float("nan"), dtype=dtype)
    vp = torch.full((Hkv, num_pages, page_size, hd), float("nan"), dtype=dtype)
    for t in range(T):
        kp[:, table[t // page_size], t % page_size] = k[t].to(dtype)
        vp[:, table[t // page_size], t % page_size] = v[t].to(dtype)
    return kp.to(DEV), vp.to(DEV), table


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("Hq,Hkv,hd,ps,window,sinks", [(4, 2, 16, 4, None, False), (6, 2, 48, 16, 21, True),
                                                        (5, 5, 80, 8, None, True), (16, 2, 128, 16, 100, False),
                                                        (3, 1, 256, 32, None, False)])
def test_attention_generic(dtype, Hq, Hkv, hd, ps, window, sinks):
    from quench6k_b200 import ops
    T = 150
    g = torch.Generator().manual_seed(Hq * 100 + hd)
    q, k, v = (torch.randn(T, h, hd, generator=g) for h in (Hq, Hkv, Hkv))
    # one far key must stand out among hundreds: scale one early key and the queries toward it
    k[3] *= 4.0
    q[-5:] += 2.0 * k[3].repeat_interleave(Hq // Hkv, 0) / k[3].norm()
    sk = torch.randn(Hq, generator=g) if sinks else None
    qd, kd, vd = (x.to(dtype) for x in (q, k, v))
    ref = P.attention(qd.double(), kd.double(), vd.double(), window, sk.double() if sinks else None, dtype == torch.bfloat16)
    kp, vp, table = _paged(kd, vd, ps, 64, dtype, seed=1)
    # two "requests" share the launch: rows 0..T-1 of request 1 (table row 1); row 0 of the table is a decoy
    bt = torch.stack([torch.flip(table, [0]), table]).to(DEV)
    rot = torch.ones(T, dtype=torch.int32, device=DEV)
    pos = torch.arange(T, dtype=torch.int32, device=DEV)
    out = ops.attention_generic(qd.to(DEV), kp, vp, bt, rot, pos, window, sk.to(DEV) if sinks else None)
    tol = 2e-5 if dtype == torch.float32 else 1.5e-2
    err = (out.double().cpu().view(T, Hq, hd) - ref).abs().max() / ref.abs().max()
    assert err <= tol, err
    # a subset of rows (decode-like: only the last position) gives the same values
    last = ops.attention_generic(qd[-1:].contiguous().to(DEV), kp, vp, bt, rot[-1:].contiguous(), pos[-1:].contiguous(), window,
                                 sk.to(DEV) if sinks else None)
    assert torch.equal(last[0], out[-1])


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("Hq,Hkv,hd,ps,norm,theta,rd,neighbours", [
    (4, 2, 16, 4, False, 10000.0, 0, False), (6, 3, 48, 8, True, 500000.0, 0, False), (2, 1, 128, 16, True, None, 0, False),
    (32, 4, 128, 16, True, 1e6, 0, False), (5, 5, 64, 8, False, 10000.0, 0, False), (3, 1, 256, 16, True, 777.0, 0, False),
    # partial rotary (the warp kernel takes multiples of 64, the block kernel the rest) and pairs of neighbours
    (8, 2, 128, 16, True, 1e4, 64, False), (4, 2, 128, 16, False, 1e4, 96, False), (6, 3, 48, 8, True, 5e4, 16, False),
    (8, 2, 128, 16, True, 1e4, 0, True), (4, 1, 64, 8, True, 1e4, 20, True), (6, 3, 48, 8, False, 5e4, 32, True)])
def test_qk_prep(dtype, Hq, Hkv, hd, ps, norm, theta, rd, neighbours):
    from quench6k_b200 import ops
    T, eps = 21, 1e-5
    rd = rd or hd
    rotary = None
    if theta is not None:
        inv = (theta ** (-(2.0 * torch.arange(rd // 2, dtype=torch.float64)) / rd)).float()
        rotary = (inv.to(DEV), rd, neighbours)

    def rotate(x, positions):
        """Plain restatement for any rotary_dim and pairing (plain_flint.rope_neox is the full-head, halves case)."""
        if rd == hd and not neighbours:
            return P.rope_neox(x, positions, theta)
        a = (positions.float()[:, None] * inv[None, :]).double()[:, None, :]
        c, s = torch.cos(a), torch.sin(a)
        out = x.clone()
        if neighbours:
            lo, hi = x[..., 0:rd:2], x[..., 1:rd:2]
            out[..., 0:rd:2], out[..., 1:rd:2] = lo * c - hi * s, hi * c + lo * s
        else:
            lo, hi = x[..., :rd // 2], x[..., rd // 2:rd]
            out[..., :rd // 2], out[..., rd // 2:rd] = lo * c - hi * s, hi * c + lo * s
        return out

    qkv = _t(T, (Hq + 2 * Hkv) * hd, seed=5)
    qn, kn = (_t(hd, seed=6) + 1.0, _t(hd, seed=7) + 1.0) if norm else (None, None)
    pos0 = 37
    pos = torch.arange(pos0, pos0 + T, dtype=torch.int32, device=DEV)
    rot = torch.zeros(T, dtype=torch.int32, device=DEV)
    nb = (pos0 + T + ps - 1) // ps
    table = torch.randperm(40)[:nb].to(torch.int32).view(1, nb).to(DEV)
    kp = torch.zeros(Hkv, 40, ps, hd, dtype=dtype, device=DEV)
    vp = torch.zeros_like(kp)
    q = ops.qk_prep(qkv, Hq, Hkv, hd, qn, kn, eps, rotary, pos, rot, table, ps, kp, vp, dtype)
    x = qkv.double().cpu()
    rq = x[:, :Hq * hd].view(T, Hq, hd)
    rk = x[:, Hq * hd:(Hq + Hkv) * hd].view(T, Hkv, hd)
    rv = x[:, (Hq + Hkv) * hd:].view(T, Hkv, hd)
    if norm:
        rq, rk = P.rmsnorm(rq, qn.double().cpu(), eps), P.rmsnorm(rk, kn.double().cpu(), eps)
    if theta is not None:
        rq, rk = rotate(rq, pos.cpu()), rotate(rk, pos.cpu())
    tol = 2e-5 if dtype == torch.float32 else 1e-2
    assert (q.double().cpu() - rq).abs().max() <= tol * rq.abs().max()
    for t in range(T):
        p = pos0 + t
        page = int(table[0, p // ps])
        assert (kp[:, page, p % ps].double().cpu() - rk[t]).abs().max() <= tol * rk.abs().max()
        assert (vp[:, page, p % ps].double().cpu() - rv[t]).abs().max() <= tol * rv.abs().max()
    # read-only layers produce the same q and leave the pages alone
    k0 = kp.clone()
    q2 = ops.qk_prep(qkv[:, :Hq * hd].contiguous(), Hq, Hkv, hd, qn, kn, eps, rotary, pos, rot, None, ps, None, None, dtype)
    assert torch.equal(q2, q) and torch.equal(kp, k0)


@pytest.mark.parametrize("rows,V", [(1, 10), (5, 384), (3, 151936), (2, 70001), (2, 8191), (9, 8192), (1, 8199), (1, 393216), (1, 400000)])
def test_argmax_and_topk_pool(rows, V):
    from quench6k_b200 import ops
    x = _t(rows, V, scale=3.0, seed=V)
    x = (x * 8).round() / 8                                              # many ties
    am = ops.argmax(x).cpu().tolist()
    for r in range(rows):
        row = x[r].cpu()
        assert am[r] == int((row == row.max()).nonzero()[0])
    for k in (1, 5, 64, 256):
        if k > V:
            continue
        ids, vals = ops.topk_pool(x, k)
        for r in range(rows):
            row = x[r].cpu().tolist()
            want = sorted(range(V), key=lambda i: (-row[i], i))[:k]
            assert ids[r].cpu().tolist() == want
            assert vals[r].cpu().tolist() == [row[i] for i in want]


def test_sample_pool_matches_the_host_sampler():
    """The choice from sorted candidate pools on the device against the host's pick_from_pool:
    greedy rows, every sampling option, pools smaller than the fetched width, rows left alone."""
    import random
    import numpy as np
    from quench6k_b200 import ops
    from quench6k_b200.sampling import SamplingParams, SplitMix64
    from quench6k_b200.sampling.sampler import ROW_RECORD, device_rows, pick_from_pool, pool_size
    rng = random.Random(11)
    for case in range(12):
        rows, V = rng.randint(1, 40), rng.choice([300, 5000])
        logits = torch.tensor([[round(rng.gauss(0, 3), rng.choice([1, 5])) for _ in range(V)] for _ in range(rows)], dtype=torch.float32)
        params = [SamplingParams(temperature=rng.choice([0.0, 0.4, 1.0, 3.0]), top_k=rng.choice([0, 1, 7, 20, 200]),
                                 top_p=rng.choice([1.0, 0.95, 0.4]), min_p=rng.choice([0.0, 0.03, 0.2])) for _ in range(rows)]
        seeds = [rng.getrandbits(64) for _ in range(rows)]
        a, b = [SplitMix64(x) for x in seeds], [SplitMix64(x) for x in seeds]
        rec = np.zeros(rows, dtype=ROW_RECORD)
        k = device_rows(params, a, V, rec)
        skip = rng.randrange(rows)
        rec[skip]["size"] = 0
        ids, vals = ops.topk_pool(logits.to(DEV), k)
        out = torch.full((rows + 3,), -5, dtype=torch.int32, device=DEV)
        got = ops.sample_pool(ids, vals, torch.from_numpy(rec.view(np.int32).reshape(rows, 8)).to(DEV), out=out).cpu().tolist()
        ids, vals = ids.cpu().numpy(), vals.cpu().numpy()
        for r in range(rows):
            n = pool_size(params[r], V)
            want = pick_from_pool(ids[r, :n], vals[r, :n], params[r], [], b[r])
            assert a[r].state == b[r].state
            assert got[r] == (want if r != skip else -5), (case, r, params[r])
        assert out[rows:].cpu().tolist() == [-5, -5, -5]


def test_kernels_refuse_what_they_cannot_do():
    from quench6k_b200 import ops
    q = torch.zeros(1, 2, 24, device=DEV)
    pages = torch.zeros(1, 2, 4, 24, device=DEV)
    z = torch.zeros(1, dtype=torch.int32, device=DEV)
    with pytest.raises(ops.KernelError, match="multiple of 16"):
        ops.attention_generic(q, pages, pages, z.view(1, 1), z, z, None, None)
    with pytest.raises(ops.KernelError, match="outside"):
        ops.topk_pool(torch.zeros(1, 1000, device=DEV), 300)
    with pytest.raises(ops.KernelError, match="CUDA device"):
        ops.argmax(torch.zeros(2, 5))
    with pytest.raises(ops.KernelError, match="dtype"):
        ops.embed(torch.zeros(2, dtype=torch.int64, device=DEV), torch.zeros(4, 4, device=DEV))


# --------------------------------------------------------------------------- tcgen05 tensor-core products
@pytest.mark.parametrize("M,N,K", [(1, 256, 64), (8, 5120, 2048), (16, 100, 72), (17, 384, 200), (70, 130, 1024),
                                   (200, 512, 136), (300, 1000, 4096), (2048, 640, 512), (5, 2048, 4096), (2048, 5120, 256),
                                   (700, 2000, 264), (1100, 2304, 1032), (1300, 2200, 512), (2048, 2048, 4096)])
def test_gemm_tc_dense(M, N, K):
    from quench6k_b200 import ops
    a, w = _t(M, K, dtype=torch.bfloat16), _t(N, K, dtype=torch.bfloat16, seed=1)
    ref = a.double().cpu() @ w.double().cpu().T
    out = ops.gemm_tc(a, w)
    assert ops.tc_status() == 0
    tol = 1e-5 * math.sqrt(K) * ref.abs().max()
    assert (out.double().cpu() - ref).abs().max() <= tol
    base = _t(M, N, seed=2)
    acc = base.clone()
    ops.gemm_tc(a, w, out=acc, accumulate=True)
    assert (acc.double().cpu() - (base.double().cpu() + ref)).abs().max() <= tol
    w2 = _t(N, K, dtype=torch.bfloat16, seed=3)
    act = ops.gemm_tc(a, w, w2=w2)
    want = P.silu(ref) * (a.double().cpu() @ w2.double().cpu().T)
    assert act.dtype == torch.bfloat16
    assert (act.double().cpu() - want).abs().max() <= 1e-2 * want.abs().max()
    assert ops.tc_status() == 0
    # a row's result does not depend on the rows beside it as long as the shape class is the same
    if M > 1:
        again = ops.gemm_tc(torch.cat([a[1:], a[:1]]).contiguous(), w)
        assert torch.equal(again[-1], out[0])


@pytest.mark.parametrize("M,N,K", [(1, 5120, 2048), (2, 2048, 4096), (1, 100, 72), (3, 77, 264), (4, 384, 1032), (1, 5, 8), (2, 33, 520)])
def test_gemv_dense(M, N, K):
    """The matrix-vector kernel for steps of one to four tokens against float64: plain store,
    accumulation, the SwiGLU epilogue; ragged row counts and widths that are no multiple of the
    256-element stride of a warp."""
    from quench6k_b200 import ops
    a, w = _t(M, K, dtype=torch.bfloat16), _t(N, K, dtype=torch.bfloat16, seed=1)
    ref = a.double().cpu() @ w.double().cpu().T
    out = ops.gemv(a, w)
    tol = 1e-5 * math.sqrt(K) * ref.abs().max()
    assert out.dtype == torch.float32 and (out.double().cpu() - ref).abs().max() <= tol
    base = _t(M, N, seed=2)
    acc = base.clone()
    ops.gemv(a, w, out=acc, accumulate=True)
    assert (acc.double().cpu() - (base.double().cpu() + ref)).abs().max() <= tol
    w2 = _t(N, K, dtype=torch.bfloat16, seed=3)
    act = ops.gemv(a, w, w2=w2)
    want = P.silu(ref) * (a.double().cpu() @ w2.double().cpu().T)
    assert act.dtype == torch.bfloat16 and (act.double().cpu() - want).abs().max() <= 1e-2 * want.abs().max()
    with pytest.raises(ops.KernelError, match="tokens"):
        ops.gemv(_t(5, K, dtype=torch.bfloat16), w)
    assert ops.gemv_preferred(1, 5120, 2048) and not ops.gemv_preferred(8, 5120, 2048) and not ops.gemv_preferred(1, 151936, 2048)


@pytest.mark.parametrize("M,N,K", [(8, 5120, 2048), (3, 4096, 512), (16, 4100, 4096), (11, 77, 520), (1, 16, 1032), (9, 40, 264), (5, 8200, 8)])
def test_gemm_skinny(M, N, K):
    """The mma.sync kernel for at most 16 tokens against float64 (its operands enter the instruction in a permuted
    order of k, which both sides must agree on): store, accumulation, SwiGLU; ragged rows, tokens and widths."""
    from quench6k_b200 import ops
    a, w = _t(M, K, dtype=torch.bfloat16), _t(N, K, dtype=torch.bfloat16, seed=1)
    ref = a.double().cpu() @ w.double().cpu().T
    out = ops.gemm_skinny(a, w)
    tol = 1e-5 * math.sqrt(K) * ref.abs().max()
    assert out.dtype == torch.float32 and (out.double().cpu() - ref).abs().max() <= tol
    base = _t(M, N, seed=2)
    acc = base.clone()
    ops.gemm_skinny(a, w, out=acc, accumulate=True)
    assert (acc.double().cpu() - (base.double().cpu() + ref)).abs().max() <= tol
    w2 = _t(N, K, dtype=torch.bfloat16, seed=3)
    act = ops.gemm_skinny(a, w, w2=w2)
    want = P.silu(ref) * (a.double().cpu() @ w2.double().cpu().T)
    assert act.dtype == torch.bfloat16 and (act.double().cpu() - want).abs().max() <= 1e-2 * want.abs().max()
    with pytest.raises(ops.KernelError, match="tokens"):
        ops.gemm_skinny(_t(17, K, dtype=torch.bfloat16), w)
    assert ops.gemm_skinny_preferred(8, 5120, 2048) and ops.gemm_skinny_preferred(1, 151936, 2048)
    assert not ops.gemm_skinny_preferred(8, 2048, 4096) and not ops.gemm_skinny_preferred(1, 5120, 2048) and not ops.gemm_skinny_preferred(17, 5120, 2048)
    # K in slices whose partial sums the caller adds: any number of slices gives the product
    for slices in (2, 3, 5):
        parts = ops.gemm_skinny(a, w, slices=slices)
        assert parts.shape == (slices, M, N)
        assert (parts.double().sum(0).cpu() - ref).abs().max() <= tol, slices
    assert ops.gemm_skinny_slices(8, 2048, 4096) == 2 and ops.gemm_skinny_slices(8, 1024, 4096) == 4
    assert ops.gemm_skinny_slices(8, 5120, 2048) == 0 and ops.gemm_skinny_slices(2, 2048, 4096) == 0 and ops.gemm_skinny_slices(8, 2048, 1024) == 0


@pytest.mark.parametrize("T,k,E,D,I", [(1, 8, 256, 2048, 512), (2, 3, 7, 264, 40), (9, 2, 5, 72, 136)])
def test_gemv_per_pair(T, k, E, D, I):
    """The same kernel with one (token, expert) pair per block row, as the decode path of the experts calls it."""
    from quench6k_b200 import ops
    x = _t(T, D, dtype=torch.bfloat16)
    wg, wu, wd = _t(E, I, D, dtype=torch.bfloat16, seed=1), _t(E, I, D, dtype=torch.bfloat16, seed=2), _t(E, D, I, dtype=torch.bfloat16, seed=3)
    g = torch.Generator().manual_seed(T)
    sel = torch.stack([torch.randperm(E, generator=g)[:k] for _ in range(T)]).to(torch.int32).to(DEV)
    act = ops.gemv(x, wg, w2=wu, pair_expert=sel.view(-1), pair_div=k)
    y = ops.gemv(act, wd, pair_expert=sel.view(-1), pair_div=1)
    assert act.shape == (T * k, I) and y.shape == (T * k, D) and y.dtype == torch.float32
    xd = x.double().cpu()
    for p in range(T * k):
        e, t = int(sel.view(-1)[p]), p // k
        a_ref = P.silu(xd[t] @ wg[e].double().cpu().T) * (xd[t] @ wu[e].double().cpu().T)
        assert (act[p].double().cpu() - a_ref).abs().max() <= 1e-2 * a_ref.abs().max()
        y_ref = act[p].double().cpu() @ wd[e].double().cpu().T
        assert (y[p].double().cpu() - y_ref).abs().max() <= 1e-5 * math.sqrt(I) * y_ref.abs().max()


def test_gemm_tc_refuses_unaligned():
    from quench6k_b200 import ops
    a, w = _t(4, 20, dtype=torch.bfloat16), _t(8, 20, dtype=torch.bfloat16)
    assert not ops.tc_supported(a, w)
    with pytest.raises(ops.KernelError, match="multiple of 8"):
        ops.gemm_tc(a, w)


@pytest.mark.parametrize("T,k,E,D,I", [(37, 3, 10, 64, 40), (8, 8, 256, 256, 128), (300, 4, 16, 136, 72), (2048, 8, 64, 128, 64)])
def test_gemm_tc_grouped(T, k, E, D, I):
    from quench6k_b200 import ops
    g = torch.Generator().manual_seed(T)
    sel = torch.stack([torch.randperm(E, generator=g)[:k] for _ in range(T)]).to(torch.int32).to(DEV)
    offsets, pair_row, row_token = ops.moe_permute(sel, E)
    pairs = T * k
    x = _t(T, D, dtype=torch.bfloat16)
    wg, wu = _t(E, I, D, dtype=torch.bfloat16, seed=1, scale=0.3), _t(E, I, D, dtype=torch.bfloat16, seed=2, scale=0.3)
    wd = _t(E, D, I, dtype=torch.bfloat16, seed=3, scale=0.3)
    avg = max(1, pairs // E)
    bt = ops.tc_token_tile(avg + avg // 2, True)
    tiles = ops.tile_list(offsets, pairs, bt)
    xs = ops.gather_rows(x, row_token)
    assert torch.equal(xs, x[row_token.long()])
    act = ops.gemm_tc(xs, wg, w2=wu, groups=tiles, bt=bt, rows=pairs)
    y = ops.gemm_tc(act, wd, groups=tiles, bt=bt, rows=pairs)
    assert ops.tc_status() == 0
    # reference: the CUDA-core kernel (itself checked against float64 above)
    simt_tiles = ops.tile_list(offsets, pairs, ops.simt_tile_rows())
    act_ref = ops.gemm_simt(x, wg, w2=wu, a_rows=row_token, groups=simt_tiles, rows=pairs)
    y_ref = ops.gemm_simt(act, wd, groups=simt_tiles, rows=pairs)
    assert (act.float() - act_ref.float()).abs().max() <= 1e-2 * act_ref.float().abs().max()
    assert (y - y_ref).abs().max() <= 1e-4 * y_ref.abs().max()


# --------------------------------------------------------------------------- tensor-core attention
@pytest.mark.parametrize("Hq,Hkv,hd,ps,window,sinks", [(32, 4, 128, 16, None, False), (8, 2, 64, 8, None, True),
                                                        (6, 2, 128, 16, 100, True), (16, 1, 64, 32, 37, False),
                                                        (5, 5, 128, 4, None, False)])
@pytest.mark.parametrize("mode", ["decode", "a few tokens", "portions"])
def test_attention_mma(Hq, Hkv, hd, ps, window, sinks, mode):
    """Several requests of different lengths in one launch; decode rows (narrow tiles of 8 or 16
    rows, keys split over CTAs and merged), a few tokens per request, or prompt portions (wide
    tiles); against float64 with one far key made to stand out.  Pages of 4 keys take the
    producer's cp.async path instead of TMA."""
    from quench6k_b200 import ops
    G = Hq // Hkv
    g = torch.Generator().manual_seed(Hq * 1000 + hd + (window or 0))
    lens = [700, 150, 333, 64, 65]
    num_pages = sum(-(-n // ps) for n in lens) + 5
    # requests 0 and 2 hold runs of consecutive pages (fetched as whole boxes), the others scattered ones
    need = [-(-n // ps) for n in lens]
    runs = {0: list(range(3, 3 + need[0])), 2: list(range(3 + need[0] + 1, 3 + need[0] + 1 + need[2]))}
    taken = set(runs[0]) | set(runs[2])
    perm = [x for x in torch.randperm(num_pages, generator=g).tolist() if x not in taken]
    kp = torch.full((Hkv, num_pages, ps, hd), float("nan"), dtype=torch.bfloat16)
    vp = torch.full((Hkv, num_pages, ps, hd), float("nan"), dtype=torch.bfloat16)
    tables, refs, qs = [], [], []
    for n in lens:
        q, k, v = (torch.randn(n, h, hd, generator=g) for h in (Hq, Hkv, Hkv))
        k[3] *= 3.0
        q[-20:] += 1.5 * k[3].repeat_interleave(G, 0) / k[3].norm()
        qd, kd, vd = (x.to(torch.bfloat16) for x in (q, k, v))
        sk = torch.randn(Hq, generator=g) if sinks else None
        if sinks and tables:
            sk = refs[0][1]                                # one sink vector per layer
        refs.append((P.attention(qd.double(), kd.double(), vd.double(), window, sk.double() if sinks else None, True), sk))
        table = runs[len(tables)] if len(tables) in runs else [perm.pop() for _ in range(-(-n // ps))]
        for t in range(n):
            kp[:, table[t // ps], t % ps] = kd[t]
            vp[:, table[t // ps], t % ps] = vd[t]
        tables.append(table)
        qs.append(qd)
    width = max(len(t) for t in tables)
    bt = torch.tensor([t + [-1] * (width - len(t)) for t in tables], dtype=torch.int32, device=DEV)
    sk = refs[0][1].to(DEV) if sinks else None
    if mode == "decode":
        q_lens = [1] * len(lens)
    elif mode == "a few tokens":
        q_lens = [min(2, max(1, 16 // G))] * len(lens) if G <= 8 else [1] * len(lens)
        q_lens[1] = 1
    else:
        q_lens = [130, 150, 33, 3, 65]
    starts = [n - ql for n, ql in zip(lens, q_lens)]
    ctx = helpers.make_context(q_lens, starts, [tables])
    q = torch.cat([qs[r][starts[r]:] for r in range(len(lens))]).contiguous().to(DEV)
    wide = ops.attention_mma_tile_rows(hd, G, max(q_lens))
    assert wide == (128 if mode == "portions" else 8 if G * max(q_lens) <= 8 else 16)
    assert ops.attention_mma_resident_ctas(hd, wide) >= torch.cuda.get_device_properties(0).multi_processor_count
    tok0, ntok, n_tiles = ctx.query_tiles(wide // G)
    want = torch.cat([refs[r][0][starts[r]:] for r in range(len(lens))]).reshape(-1, Hq * hd)
    for max_splits in (1, 4, 64):
        out = ops.attention_mma(q, kp.to(DEV), vp.to(DEV), bt, ctx.req_of_token, ctx.positions, tok0, ntok, wide, window, sk,
                                max_splits=max_splits, min_tiles=1)
        err = (out.double().cpu() - want).abs().max() / want.abs().max()
        assert err <= 1.5e-2, (max_splits, err)
    gen = ops.attention_generic(q, kp.to(DEV), vp.to(DEV), bt, ctx.req_of_token, ctx.positions, window, sk)
    assert (out.float() - gen.float()).abs().max() <= 2e-2 * gen.float().abs().max()
    # a plan made once and handed in, with a budget of CTAs that the long request gets most of
    plan = ops.attention_plan(ctx.positions, ctx.req_of_token, tok0, ntok, window, n_work=n_tiles + 9, min_per=2)
    out = ops.attention_mma(q, kp.to(DEV), vp.to(DEV), bt, ctx.req_of_token, ctx.positions, tok0, ntok, wide, window, sk, plan=plan)
    err = (out.double().cpu() - want).abs().max() / want.abs().max()
    assert err <= 1.5e-2, ("plan", err)


@pytest.mark.parametrize("Hq,Hkv,hd,ps,window,sinks,qk_norm,rd", [(32, 4, 128, 16, None, False, True, 128), (8, 2, 64, 8, None, True, True, 64),
                                                                   (6, 2, 128, 16, 100, True, False, 64), (16, 1, 64, 32, 37, False, True, 0),
                                                                   (5, 5, 128, 4, None, False, True, 128), (12, 3, 128, 64, None, False, True, 128),
                                                                   (4, 2, 64, 16, 50, True, True, 64)])
@pytest.mark.parametrize("few", [False, True, "eight"])
def test_attention_mma_prepares_q_and_keys(Hq, Hkv, hd, ps, window, sinks, qk_norm, rd, few):
    """The narrow tiles making q and the new keys themselves, from the FP32 q/k/v product: the
    pages afterwards hold the bits qk_prep writes, and the output is that of qk_prep followed by
    the kernel.  The new positions' rows of the pages hold NaN before; with two tokens a request,
    one request's tokens lie on both sides of a key tile's edge (positions 63 and 64), which with
    many splits are different CTAs' key tiles; the product then comes as three split-K slices."""
    from quench6k_b200 import ops
    G = Hq // Hkv
    g = torch.Generator().manual_seed(Hq * 1000 + hd + (window or 0) + rd)
    lens = [700, 150, 333, 64, 65]
    if few == "eight" and G > 2:
        pytest.skip("eight tokens to a tile need groups of at most two heads")
    per = 8 if few == "eight" else min(2, max(1, 16 // G)) if few else 1      # eight: as many as the kernel prepares
    q_lens = [per] * len(lens)
    q_lens[1] = 1
    starts = [n - ql for n, ql in zip(lens, q_lens)]
    num_pages = sum(-(-n // ps) for n in lens) + 5
    perm = torch.randperm(num_pages, generator=g).tolist()
    kp = torch.full((Hkv, num_pages, ps, hd), float("nan"), dtype=torch.bfloat16)
    vp = torch.full((Hkv, num_pages, ps, hd), float("nan"), dtype=torch.bfloat16)
    tables = []
    for n, start in zip(lens, starts):
        table = [perm.pop() for _ in range(-(-n // ps))]
        for t in range(start):                               # the keys of earlier steps; this step's rows stay NaN
            kp[:, table[t // ps], t % ps] = torch.randn(Hkv, hd, generator=g).to(torch.bfloat16)
            vp[:, table[t // ps], t % ps] = torch.randn(Hkv, hd, generator=g).to(torch.bfloat16)
        tables.append(table)
    width = max(len(t) for t in tables)
    bt = torch.tensor([t + [-1] * (width - len(t)) for t in tables], dtype=torch.int32, device=DEV)
    ctx = helpers.make_context(q_lens, starts, [tables])
    T = sum(q_lens)
    if few:                                                  # split-K partial products, which both kernels sum in order
        qkv = (torch.randn(3, T, (Hq + 2 * Hkv) * hd, generator=g) * 0.9).to(DEV)
    else:                                                    # rows with a pitch of their own
        qkv = (torch.randn(T, (Hq + 2 * Hkv) * hd + 6, generator=g) * 1.5).to(DEV)[:, :(Hq + 2 * Hkv) * hd]
    qn = (1 + 0.1 * torch.randn(hd, generator=g)).to(DEV) if qk_norm else None
    kn = (1 + 0.1 * torch.randn(hd, generator=g)).to(DEV) if qk_norm else None
    rotary = None
    if rd:
        inv = (10000.0 ** (-torch.arange(0, rd, 2, dtype=torch.float64) / rd)).to(torch.float32).to(DEV)
        rotary = (inv, rd, False)
    sk = torch.randn(Hq, generator=g).to(DEV) if sinks else None
    rows = ops.attention_mma_tile_rows(hd, G, max(q_lens))
    assert rows in (8, 16) and ops.attention_mma_prepares(hd, G, rows, rd, False)
    assert not ops.attention_mma_prepares(hd, G, 128, rd, False) and not ops.attention_mma_prepares(hd, G, rows, 32, False)
    assert not ops.attention_mma_prepares(hd, 1, 16, rd, False)             # sixteen tokens to a tile: qk_prep's work
    tok0, ntok, n_tiles = ctx.query_tiles(rows // G)
    k1, v1 = kp.to(DEV), vp.to(DEV)
    q = ops.qk_prep(qkv.contiguous(), Hq, Hkv, hd, qn, kn, 1e-5, rotary, ctx.positions, ctx.req_of_token, bt, ps, k1, v1, torch.bfloat16)
    prepare = {"qkv": qkv, "heads": Hq, "q_norm": qn, "k_norm": kn, "eps": 1e-5, "rotary": rotary, "write": True}
    for max_splits in (1, 4, 64):
        want = ops.attention_mma(q, k1, v1, bt, ctx.req_of_token, ctx.positions, tok0, ntok, rows, window, sk, max_splits=max_splits, min_tiles=1)
        k2, v2 = kp.to(DEV), vp.to(DEV)
        got = ops.attention_mma(None, k2, v2, bt, ctx.req_of_token, ctx.positions, tok0, ntok, rows, window, sk, max_splits=max_splits,
                                min_tiles=1, prepare=prepare)
        assert ops.tc_status() == 0
        assert torch.equal(k2.view(torch.int16), k1.view(torch.int16)) and torch.equal(v2.view(torch.int16), v1.view(torch.int16)), max_splits
        assert not torch.isnan(got.float()).any()
        assert (got.float() - want.float()).abs().max() <= 1e-2 * want.float().abs().max(), max_splits
    # a layer that reads another layer's cache: q alone is made; the pages stay as they are
    got = ops.attention_mma(None, k1, v1, bt, ctx.req_of_token, ctx.positions, tok0, ntok, rows, window, sk, max_splits=4, min_tiles=1,
                            prepare=dict(prepare, qkv=qkv[..., :Hq * hd], write=False))
    assert (got.float() - want.float()).abs().max() <= 1e-2 * want.float().abs().max()
    assert torch.equal(k2.view(torch.int16), k1.view(torch.int16))


@pytest.mark.parametrize("window", [None, 300])
@pytest.mark.parametrize("n_work,min_per", [(7, 2), (8, 1), (40, 2), (296, 2), (1000, 3)])
def test_attention_plan_shares_the_key_tiles(window, n_work, min_per):
    """The device-made plan of the key splits: every tile's key tiles are covered once by its
    parts, the parts are consecutive work items, no more work items are used than given, and a
    request deep in its context gets more of them than the others."""
    from quench6k_b200 import ops
    q_lens = [1, 2, 1, 40, 1, 1, 2]
    starts = [70000, 130, 0, 5000, 63, 64, 2047]
    tables = [[list(range(-(-(a + n) // 16))) for a, n in zip(starts, q_lens)]]
    ctx = helpers.make_context(q_lens, starts, tables)
    tok0, ntok, n_tiles = ctx.query_tiles(16)
    work, tiles = ops.attention_plan(ctx.positions, ctx.req_of_token, tok0, ntok, window, n_work, min_per)
    work, tiles = work.cpu().tolist(), tiles.cpu().tolist()
    assert len(work) == max(n_work, n_tiles) and len(tiles) == n_tiles
    pos = ctx.positions.cpu().tolist()
    req = ctx.req_of_token.cpu().tolist()
    used, biggest = 0, {}
    for i, (t0, nt, parts, w0) in enumerate(tiles):
        assert (t0, nt) == (tok0[i].item(), ntok[i].item())
        first, last = pos[t0], pos[t0] + nt - 1
        lo = max(0, first - window + 1) if window else 0
        n = last // 64 + 1 - lo // 64
        covered = 0
        for s in range(parts):
            a, b = work[w0 + s][:4], work[w0 + s][4:]
            assert a == [t0, nt, first, req[t0]] and b[:3] == [s, parts, w0]
            each = b[3]
            covered += min(each, n - s * each)
            assert n - s * each > 0                                  # no part without keys
            assert each >= min(min_per, n)
        assert covered == n
        used = max(used, w0 + parts)
        biggest[i] = parts
    live = [w for w in work if w[0] >= 0]
    assert len(live) == sum(biggest.values()) and used <= len(work)
    if n_work >= 40 and window is None:
        assert biggest[0] == max(biggest.values()) and biggest[0] > 4 * biggest[2]      # 70,000 keys against one


@pytest.mark.parametrize("scoring,renorm", [("softmax", True), ("sigmoid", False)])
@pytest.mark.parametrize("T,E,k,D,I", [(1, 256, 8, 2048, 512), (8, 256, 8, 2048, 512), (16, 256, 8, 2048, 512), (8, 64, 6, 256, 128), (16, 10, 3, 72, 40), (2, 32, 4, 1024, 256),
                                       (3, 16, 2, 640, 1024), (5, 300, 7, 128, 64), (4, 704, 6, 2048, 64), (12, 520, 5, 3072, 64)])
def test_decode_moe_path(scoring, renorm, T, E, k, D, I):
    """router_small + per-pair expert tiles against float64.  The first and two of the small sizes have
    so few pairs that the pair products slice K over CTAs (both epilogues).  The last two have more
    experts per CTA of the router's cluster than fit its shared memory at once: their rows go through
    one buffer, chunk after chunk (32 rows of 2,048, 16 rows of 3,072)."""
    from quench6k_b200 import ops
    x = _t(T, D, dtype=torch.bfloat16)
    wr = _t(E, D, dtype=torch.bfloat16, seed=1, scale=0.02)      # small: a saturated sigmoid would tie in FP32
    wg, wu = _t(E, I, D, dtype=torch.bfloat16, seed=2, scale=0.2), _t(E, I, D, dtype=torch.bfloat16, seed=3, scale=0.2)
    wd = _t(E, D, I, dtype=torch.bfloat16, seed=4, scale=0.2)
    sel_e, sel_w, order = ops.router_small(x, wr, k, scoring, renorm)
    flat = sel_e.flatten().cpu()
    assert torch.equal(order.cpu().long(), torch.sort(flat, stable=True).indices)
    logits = x.double().cpu() @ wr.double().cpu().T
    ref_e, ref_w = P.route(logits, scoring, k, renorm)
    assert torch.equal(sel_e.cpu().long(), ref_e)
    assert (sel_w.double().cpu() - ref_w).abs().max() <= 1e-4 * ref_w.abs().max()
    again_e, again_w, _ = ops.router_small(x, wr, k, scoring, renorm)       # the ticket was left ready
    assert torch.equal(again_e, sel_e) and torch.equal(again_w, sel_w)
    act = ops.gemm_tc_pairs(x, wg, sel_e, k, w2=wu, order=order)
    y = ops.gemm_tc_pairs(act, wd, sel_e, 1, order=order)
    assert torch.equal(act, ops.gemm_tc_pairs(x, wg, sel_e, k, w2=wu))      # the order of work does not change a value
    assert ops.tc_status() == 0
    for p in range(T * k):
        e, t = int(sel_e.flatten()[p]), p // k
        xa = x[t].double().cpu()
        a_ref = P.silu(wg[e].double().cpu() @ xa) * (wu[e].double().cpu() @ xa)
        assert (act[p].double().cpu() - a_ref).abs().max() <= 1e-2 * a_ref.abs().max() + 1e-9
        y_ref = wd[e].double().cpu() @ act[p].double().cpu()
        assert (y[p].double().cpu() - y_ref).abs().max() <= 1e-4 * y_ref.abs().max() + 1e-9
    h = _t(T, D, seed=9)
    want = h.double().cpu() + (sel_w.double().cpu()[:, :, None] * y.double().cpu().view(T, k, D)).sum(1)
    ops.combine(y, None, sel_w, h)
    assert (h.double().cpu() - want).abs().max() <= 1e-5 * want.abs().max()


@pytest.mark.parametrize("Hq,Hkv,ps,window,sinks", [(32, 4, 16, None, False), (8, 1, 8, None, True), (6, 2, 32, 100, True),
                                                     (16, 16, 64, 37, False), (5, 1, 128, None, False)])
def test_attention_tc(Hq, Hkv, ps, window, sinks):
    """Prompt portions of several requests (some continuing from a cache) through the tcgen05
    attention kernel, against float64 with one far key made to stand out."""
    from quench6k_b200 import ops
    hd, G = 128, Hq // Hkv
    g = torch.Generator().manual_seed(Hq * 1000 + ps + (window or 0))
    lens = [700, 150, 333, 64, 129]
    num_pages = sum(-(-n // ps) for n in lens) + 5
    # requests 0 and 2 hold runs of consecutive pages (fetched as whole boxes), the others scattered ones
    need = [-(-n // ps) for n in lens]
    runs = {0: list(range(3, 3 + need[0])), 2: list(range(3 + need[0] + 1, 3 + need[0] + 1 + need[2]))}
    taken = set(runs[0]) | set(runs[2])
    perm = [x for x in torch.randperm(num_pages, generator=g).tolist() if x not in taken]
    kp = torch.full((Hkv, num_pages, ps, hd), float("nan"), dtype=torch.bfloat16)
    vp = torch.full((Hkv, num_pages, ps, hd), float("nan"), dtype=torch.bfloat16)
    tables, refs, qs = [], [], []
    sk = torch.randn(Hq, generator=g) if sinks else None
    for n in lens:
        q, k, v = (torch.randn(n, h, hd, generator=g) for h in (Hq, Hkv, Hkv))
        k[3] *= 3.0
        q[-20:] += 1.5 * k[3].repeat_interleave(G, 0) / k[3].norm()
        qd, kd, vd = (x.to(torch.bfloat16) for x in (q, k, v))
        refs.append(P.attention(qd.double(), kd.double(), vd.double(), window, sk.double() if sinks else None, True))
        table = runs[len(tables)] if len(tables) in runs else [perm.pop() for _ in range(-(-n // ps))]
        for t in range(n):
            kp[:, table[t // ps], t % ps] = kd[t]
            vp[:, table[t // ps], t % ps] = vd[t]
        tables.append(table)
        qs.append(qd)
    width = max(len(t) for t in tables)
    bt = torch.tensor([t + [-1] * (width - len(t)) for t in tables], dtype=torch.int32, device=DEV)
    q_lens = [700, 150, 33, 3, 129]
    starts = [n - ql for n, ql in zip(lens, q_lens)]
    ctx = helpers.make_context(q_lens, starts, [tables])
    q = torch.cat([qs[r][starts[r]:] for r in range(len(lens))]).contiguous().to(DEV)
    want = torch.cat([refs[r][starts[r]:] for r in range(len(lens))]).reshape(-1, Hq * hd)
    for zigzag in (False, True):                 # neighbours together; a late tile with an early one
        tok0, ntok, n_tiles = ctx.query_tile_pairs(ops.attention_tc_tile_tokens(G), zigzag)
        out = ops.attention_tc(q, kp.to(DEV), vp.to(DEV), bt, ctx.req_of_token, ctx.positions, tok0, ntok, window,
                               sk.to(DEV) if sinks else None)
        assert ops.tc_status() == 0
        err = (out.double().cpu() - want).abs().max() / want.abs().max()
        assert err <= 1.5e-2, (zigzag, err)
    # the step in two parts that write one output: the requests with more than half a tile of tokens here, the others
    # through the kernel that splits the keys (its partial sums sized for the rows it covers)
    tile = ops.attention_tc_tile_tokens(G)
    cut = tile // 2
    count, row0, row1, most, reach = ctx.short_requests(cut)
    wide = ops.attention_mma_tile_rows(hd, G, most)
    if count and wide:
        assert count == sum(1 for n in q_lens if n <= cut) and (row0, row1) == (sum(q_lens[:2]) if q_lens[2] <= cut else sum(q_lens[:3]), sum(q_lens[:4]))
        out = torch.full((q.shape[0], Hq * hd), float("nan"), dtype=torch.bfloat16, device=DEV)
        tok0, ntok, n_pairs = ctx.query_tile_pairs(tile, False, more_than=cut)
        ops.attention_tc(q, kp.to(DEV), vp.to(DEV), bt, ctx.req_of_token, ctx.positions, tok0, ntok, window, sk.to(DEV) if sinks else None, out=out)
        assert torch.isnan(out[row0:row1].float()).any() and not torch.isnan(out[:row0].float()).any()
        s0, sn, n_short = ctx.query_tiles(wide // G, at_most=cut)
        ops.attention_mma(q, kp.to(DEV), vp.to(DEV), bt, ctx.req_of_token, ctx.positions, s0, sn, wide, window,
                          sk.to(DEV) if sinks else None, max_splits=3, min_tiles=1, out=out)
        assert ops.tc_status() == 0
        err = (out.double().cpu() - want).abs().max() / want.abs().max()
        assert err <= 1.5e-2, ("two kernels", err)


def test_a_bounded_wait_that_runs_out_is_recorded_and_the_device_stays_usable():
    """Every spin of the kernels on an mbarrier has a limit.  A kernel that waits on a barrier nothing arrives on
    (limit: two million cycles, about a millisecond) comes back with the run-out recorded, having waited at least
    that long, and the next kernels run as before."""
    from quench6k_b200 import ops
    status, waited = ops.selftest_wait_runs_out(2_000_000)
    assert status == 1 and 2_000_000 <= waited < 50_000_000
    x = _t(3, 1000, seed=5)
    assert torch.equal(ops.argmax(x).long().cpu(), x.argmax(-1).cpu())
    assert ops.tc_status() == 0                                  # no product kernel's wait has run out in this process

