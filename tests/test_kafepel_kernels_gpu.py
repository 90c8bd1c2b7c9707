"""The kernels of sigmoid attention, retention, routing and side-by-side mixers against their plain statements
(tests/plain_ops.py) at odd sizes, and attention inputs built so that one key decides the result."""

from __future__ import annotations

from types import SimpleNamespace

import numpy as np
import pytest
import torch

import plain_ops

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _ops():
    from llmserve_triton_kernels_b200 import ops

    return ops


def close(a, b, tol, what):
    a, b = a.float().cpu(), b.float().cpu()
    err = float((a - b).abs().max()) / max(1e-9, float(b.abs().max()))
    assert err <= tol, f"{what}: relative error {err:.3e} > {tol:.1e}"


def paged_batch(lens, news, page_size, extra_pages=3, seed=0):
    """A step's arrays for requests holding ``lens`` tokens after bringing ``news`` of them, over shuffled pages."""
    g = torch.Generator().manual_seed(seed)
    R, N = len(lens), sum(news)
    cu = np.concatenate([[0], np.cumsum(news)]).astype(np.int32)
    pos = np.concatenate([np.arange(n - k, n) for n, k in zip(lens, news)]).astype(np.int32)
    owner = np.repeat(np.arange(R), news).astype(np.int32)
    per = [-(-n // page_size) for n in lens]
    pages = sum(per) + extra_pages
    perm = torch.randperm(pages, generator=g).tolist()
    table = np.zeros((R, max(per)), np.int32)
    k = 0
    for r in range(R):
        for i in range(per[r]):
            table[r, i] = perm[k]
            k += 1
    slots = np.array([table[owner[t], pos[t] // page_size] * page_size + pos[t] % page_size for t in range(N)], np.int32)
    T = lambda a: torch.tensor(a, device=DEV)  # noqa: E731
    ctx = SimpleNamespace(positions=T(pos), token_request=T(owner), cu_tokens=T(cu), context_lens=T(np.array(lens, np.int32)),
                          max_context_len=max(lens), max_query_len=max(news), num_requests=R, num_tokens=N)
    return ctx, T(table), T(slots), pages


SHAPES = [(8, 2, 24, 40, 24, 16), (3, 1, 10, 6, 4, 8), (40, 8, 16, 32, 8, 16), (4, 4, 128, 128, 64, 4), (1, 1, 2, 1, 2, 1), (5, 5, 7, 3, 0, 3),
          (6, 2, 48, 80, 32, 16), (32, 8, 64, 64, 64, 16), (24, 24, 32, 16, 16, 8)]


@pytest.mark.parametrize("general", [False, True])
@pytest.mark.parametrize("dtype,tol", [(torch.float32, 2e-5), (torch.bfloat16, 2e-2)])
@pytest.mark.parametrize("H,KV,D,V,rot,page_size", SHAPES)
def test_prepare_and_attention_against_plain(H, KV, D, V, rot, page_size, dtype, tol, general, monkeypatch):
    """``general``: the kernel for any sizes also where the tensor-core kernel would run (bfloat16, lanes in sixteens)."""
    ops = _ops()
    if general and dtype == torch.float32:
        pytest.skip("float32 always runs the general kernel")
    monkeypatch.setattr(ops, "_FORCE_GENERIC_ATTENTION", general)
    torch.manual_seed(H * 100 + D)
    ctx, table, slots, pages = paged_batch([37, 1, 200, 530], [5, 1, 200, 2], page_size)
    N = ctx.num_tokens
    pool = (torch.randn(pages, 2, KV, page_size, max(D, V), device=DEV) * 0.5).to(dtype)
    proj = torch.randn(N, (H + KV) * D + KV * V + 7, device=DEV)
    freq = torch.rand(rot // 2, device=DEV) if rot else None
    qw, kw = torch.randn(H * D, device=DEV), torch.randn(KV * D, device=DEV)
    kwargs = dict(heads=H, kv_heads=KV, dim=D, value_dim=V, freq=freq, q_weight=qw, k_weight=kw, eps=1e-5, slot_map=slots)
    p1, p2 = pool.clone(), pool.clone()
    q1 = ops.qk_prepare(proj, ctx.positions, pool=p1, **kwargs)
    q2 = plain_ops.qk_prepare(proj, ctx.positions, pool=p2, **kwargs)
    close(q1, q2, tol, "prepared queries")
    close(p1, p2, tol, "keys and values in their pages")
    bias, mix = torch.randn(H, device=DEV), torch.randn(H, H, device=DEV)
    common = dict(num_heads=H, num_kv_heads=KV, key_dim=D, value_dim=V, scale=0.2)
    for what, more in (("cap, bias, mixed heads", dict(softcap=5.0, head_bias=bias, head_mix=mix)), ("bare", {}), ("window", dict(window=33, head_mix=mix))):
        close(ops.sigmoid_attention(q2, p2, table, ctx, **common, **more), plain_ops.sigmoid_attention(q2, p2, table, ctx, **common, **more), tol, what)
    # the same rows as single tokens of a small step: the contexts are shared out over CTAs and summed
    rows = [4, 5, 205, 207]
    few = SimpleNamespace(positions=ctx.positions[rows].contiguous(), token_request=ctx.token_request[rows].contiguous(), max_context_len=530,
                          max_query_len=1, num_requests=4, num_tokens=4, context_lens=ctx.context_lens,
                          cu_tokens=torch.arange(5, dtype=torch.int32, device=DEV), host_cu_tokens=[0, 1, 2, 3, 4])
    more = dict(softcap=5.0, head_bias=bias, head_mix=mix)
    a = ops.sigmoid_attention(q2[rows].contiguous(), p2, table, few, **common, **more)
    close(a, plain_ops.sigmoid_attention(q2, p2, table, ctx, **common, **more)[rows], tol, "keys shared out")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("general", [False, True])
@pytest.mark.parametrize("news", [[600, 1, 1], [1, 1, 1], [64, 2, 1]])
def test_one_key_decides(news, dtype, general, monkeypatch):
    """Keys are built from the three base-9 digits of their position (a third of a unit vector per digit), so that a query
    66 times key j scores 66 on key j and at most 44 on any other; with a bias of -52 per head only key j is left with a
    weight.  The chosen key: the one at position 0, one 1 / 7 / 8 back (page borders), 255 / 256 / 257 back (the border of a
    stretch of keys), and the query's own.  The output must be that key's value row, through the mixing matrix."""
    ops = _ops()
    monkeypatch.setattr(ops, "_FORCE_GENERIC_ATTENTION", general)
    H, KV, D, V, page_size = 4, 2, 32, 16, 8
    lens = [600, 523, 300]
    ctx, table, slots, pages = paged_batch(lens, news, page_size, seed=3)
    pool = torch.zeros(pages, 2, KV, page_size, D, device=DEV, dtype=dtype)
    j = torch.arange(max(lens))
    code = torch.zeros(max(lens), D)
    for digit in range(3):
        code[j, 9 * digit + (j // 9 ** digit) % 9] = 3 ** -0.5
    vals = {r: torch.randn(n, KV, V) for r, n in enumerate(lens)}
    host_table = table.cpu()
    for r, n in enumerate(lens):
        for jj in range(n):
            page, off = int(host_table[r, jj // page_size]), jj % page_size
            pool[page, 0, :, off] = code[jj].to(dtype)
            pool[page, 1, :, off, :V] = vals[r][jj].to(dtype)
    mix = torch.eye(H, device=DEV) + 0.25
    bias = torch.full((H,), -52.0, device=DEV)
    positions, owner = ctx.positions.cpu().tolist(), ctx.token_request.cpu().tolist()
    weight = (mix.cpu() @ torch.full((H,), float(torch.sigmoid(torch.tensor(14.0)))))
    for back in (0, 1, 7, 8, 255, 256, 257, None):
        target = [0 if back is None else max(0, pos - back) for pos in positions]
        q = (66.0 * code[target])[:, None, :].expand(-1, H, -1).reshape(ctx.num_tokens, H * D).to(DEV)
        want = torch.stack([torch.stack([weight[h] * vals[owner[t]][target[t]][h // (H // KV)].to(dtype).float() for h in range(H)])
                            for t in range(ctx.num_tokens)])
        out = ops.sigmoid_attention(q.to(dtype).contiguous(), pool, table, ctx, num_heads=H, num_kv_heads=KV, key_dim=D, value_dim=V,
                                    scale=1.0, softcap=None, head_bias=bias, head_mix=mix)
        err = (out.float().cpu().view(-1, H, V) - want).abs().max(-1).values.max(-1).values
        bad = torch.nonzero(err > 0.06)
        assert not len(bad), f"key {back} back: first wrong query is token {int(bad[0])} at position {positions[int(bad[0])]}: {float(err.max()):.3f}"


@pytest.mark.parametrize("H,D,V", [(4, 32, 64), (3, 10, 14), (1, 1, 1), (2, 130, 17), (5, 64, 256), (2, 256, 20)])
@pytest.mark.parametrize("vdtype", [torch.float32, torch.bfloat16])
def test_retention_scan_and_head_norm(H, D, V, vdtype):
    ops = _ops()
    torch.manual_seed(D)
    news = [5, 1, 120, 2]
    cu = torch.tensor(np.concatenate([[0], np.cumsum(news)]).astype(np.int32), device=DEV)
    N = sum(news)
    q, k = torch.randn(N, H * D + 3, device=DEV)[:, : H * D], torch.randn(N, H * D, device=DEV) * D ** -0.5
    v = torch.randn(N, H * V + 5, device=DEV).to(vdtype)[:, : H * V]
    decay = torch.rand(H, device=DEV) * 0.1 + 0.9
    s1 = torch.randn(6, H, D, V, device=DEV)
    s2 = s1.clone()
    slots = torch.tensor([3, 0, 5, 1], dtype=torch.int32, device=DEV)
    o1 = ops.retention_scan(q, k, v, decay, s1, slots, cu, 4, H, D, V)
    o2 = plain_ops.retention_scan(q, k, v, decay, s2, slots, cu, 4, H, D, V)
    close(o1, o2, 1e-4, "outputs")
    close(s1, s2, 1e-4, "states")
    s5, s6 = s1.clone(), s2.clone()  # the form for steps of few tokens a request (16 columns a CTA)
    few_cu = torch.tensor([0, 3, 4, 9, 11], dtype=torch.int32, device=DEV)
    close(ops.retention_scan(q[:11], k[:11], v[:11], decay, s5, slots, few_cu, 4, H, D, V, max_query_len=5),
          plain_ops.retention_scan(q[:11], k[:11], v[:11], decay, s6, slots, few_cu, 4, H, D, V), 1e-4, "outputs, few tokens")
    close(s5, s6, 1e-4, "states, few tokens")
    # the same with the long request shared out over CTAs in stretches (the others are shorter than a stretch's turn of eight)
    s3 = s1.clone().copy_(torch.randn(6, H, D, V, device=DEV))
    s4 = s3.clone()
    o3 = ops.retention_scan(q, k, v, decay, s3, slots, cu, 4, H, D, V, max_query_len=640)
    o4 = plain_ops.retention_scan(q, k, v, decay, s4, slots, cu, 4, H, D, V)
    close(o3, o4, 1e-4, "outputs, stretches")
    close(s3, s4, 1e-4, "states, stretches")
    assert torch.equal(s1[[2, 4]], s2[[2, 4]])  # slots of no request are left alone
    gate = torch.randn(N, H * V + 3, device=DEV).to(vdtype)[:, : H * V]
    for kind in ("silu", "sigmoid"):
        close(ops.head_norm_gate(o2, gate, 1e-6, kind, vdtype), plain_ops.head_norm_gate(o2, gate, 1e-6, kind, vdtype), 2e-2 if vdtype == torch.bfloat16 else 1e-5, kind)
    close(ops.head_norm_gate(o2, None, None, out_dtype=torch.float32), o2.reshape(N, -1), 1e-6, "no norm, no gate")


@pytest.mark.parametrize("E,top,ff,shared", [(12, 3, 16, 24), (5, 5, 7, 0), (70, 2, 3, 9), (1, 1, 8, 8), (33, 32, 2, 0)])
def test_routing_and_expert_weights(E, top, ff, shared):
    ops = _ops()
    torch.manual_seed(E)
    N = 77
    z = torch.randn(N, E + 1, device=DEV) * 2
    corr = torch.randn(E, device=DEV) * 0.2
    close(ops.route_topk(z, corr, E, top, 2.5, False, True), plain_ops.route_topk(z, corr, E, top, 2.5, False, True), 1e-5, "weights")
    close(ops.route_topk(z, None, E, top, 1.0, True, False), plain_ops.route_topk(z, None, E, top, 1.0, True, False), 1e-5, "renormalised")
    w = ops.route_topk(z, corr, E, top, 2.5, False, True)
    assert bool(((w[:, :E] != 0).sum(-1) == top).all())
    # the correction decides the choice and stays out of the weights: a large one on expert 0 makes it chosen with its own score
    big = corr.clone()
    big[0] = 10.0
    w = ops.route_topk(z, big, E, top, 1.0, False, False)
    close(w[:, 0], torch.softmax(z[:, :E], -1)[:, 0], 1e-5, "the chosen expert's weight is its score")
    # the router's product and the choice in one kernel, from 32-bit and from bfloat16 rows with a pitch
    for K in (40, 256):
        wr = torch.randn(E + 1, K, device=DEV)
        for dtype in (torch.float32, torch.bfloat16):
            h = torch.randn(N, K + 8, device=DEV).to(dtype)[:, :K]
            zz = h.float() @ wr.t()
            margin = (zz[:, :E].softmax(-1) + corr).sort(-1).values
            sure = (margin[:, 1:] - margin[:, :-1]).min(-1).values > 1e-4 if E > 1 else torch.ones(N, dtype=torch.bool, device=DEV)
            got, ref = ops.route(h, wr, corr, E, top, 2.5, False, True), plain_ops.route(h, wr, corr, E, top, 2.5, False, True)
            close(got[sure], ref[sure], 1e-4, f"route K={K} {dtype}")
    for dtype, tol in ((torch.float32, 1e-5), (torch.bfloat16, 2e-2)):
        x = torch.randn(N, E * ff + shared, device=DEV).to(dtype)
        w = plain_ops.route_topk(z, corr, E, top, 2.5, False, True)
        for act in ("relu2", "silu"):
            close(ops.expert_act_scale(x, w, E, ff, act), plain_ops.expert_act_scale(x, w, E, ff, act), tol, act)


def test_branches_meet_normed_and_weighted():
    ops = _ops()
    torch.manual_seed(1)
    xs = [torch.randn(33, 200, device=DEV) * s for s in (1, 5, 0.1, 30)]
    ws = [torch.randn(200, device=DEV) for _ in xs]
    for count in (1, 2, 3, 4):
        close(ops.branch_norm_sum(xs[:count], ws[:count], 1e-6, 1 / count), plain_ops.branch_norm_sum(xs[:count], ws[:count], 1e-6, 1 / count), 1e-5, f"{count} branches")


@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16])
def test_branches_meet_in_the_stream_and_are_normed(out_dtype):
    ops = _ops()
    torch.manual_seed(2)
    for c in (200, 2048):
        xs = [torch.randn(19, c, device=DEV) * s for s in (1, 5)]
        ws = [torch.randn(c, device=DEV) for _ in xs]
        wn = torch.randn(c, device=DEV)
        r1 = torch.randn(19, c, device=DEV)
        r2 = r1.clone()
        pending = ops.BranchSum(xs, ws, 1e-6, 0.5)
        a = ops.branch_sum_rmsnorm(pending, r1, wn, 1e-5, out_dtype)
        b = plain_ops.branch_sum_rmsnorm(pending, r2, wn, 1e-5, out_dtype)
        close(r1, r2, 1e-5, "the stream")
        close(a, b, 1e-5 if out_dtype == torch.float32 else 1e-2, "the normed rows")
        close(pending.materialize(), plain_ops.branch_norm_sum(xs, ws, 1e-6, 0.5), 1e-5, "as a tensor")
