"""Attention-side kernels against fp32 PyTorch restatements."""

import pytest
import torch


pytestmark = pytest.mark.gpu


def _ref_rope(x, pos, theta):
    # x [rows, heads, d] fp32, rotate-half convention
    d = x.shape[-1]
    inv = theta ** (-torch.arange(0, d, 2, device=x.device, dtype=torch.float32) / d)
    ang = pos.float()[:, None] * inv[None, :]
    cos, sin = ang.cos()[:, None, :], ang.sin()[:, None, :]
    x1, x2 = x[..., : d // 2], x[..., d // 2:]
    return torch.cat([x1 * cos - x2 * sin, x2 * cos + x1 * sin], -1)


def _ref_headnorm(x, w, eps):
    n = x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps)
    return (n.bfloat16().float() * w.float()).bfloat16().float()


@pytest.mark.parametrize("d,hq,hkv", [(128, 16, 8), (64, 4, 2), (128, 32, 4)])
@pytest.mark.parametrize("use_norm", [True, False])
def test_rope_qknorm_kvwrite(d, hq, hkv, use_norm):
    from crosspool_b200.ops import attention as A

    torch.manual_seed(0)
    rows, page, pages = 37, 16, 12
    qkv = torch.randn(rows, (hq + 2 * hkv) * d, device="cuda").bfloat16()
    pos = torch.randint(0, 30000, (rows,), device="cuda", dtype=torch.int32)
    slots = torch.randperm(page * pages, device="cuda")[:rows].int()
    slots[5] = -1
    qn = (1 + 0.1 * torch.randn(d, device="cuda")).bfloat16() if use_norm else None
    kn = (1 + 0.1 * torch.randn(d, device="cuda")).bfloat16() if use_norm else None
    kc = torch.zeros(pages, page, hkv, d, device="cuda", dtype=torch.bfloat16)
    vc = torch.zeros_like(kc)
    q_out = torch.empty(rows, hq, d, device="cuda", dtype=torch.bfloat16)
    A.rope_kv_write(qkv, q_out, kc, vc, pos, slots, q_heads=hq, kv_heads=hkv, head_dim=d, theta=1e6,
                    q_norm=qn, k_norm=kn)
    x = qkv.float().view(rows, hq + 2 * hkv, d)
    q, k, v = x[:, :hq], x[:, hq:hq + hkv], x[:, hq + hkv:]
    if use_norm:
        q, k = _ref_headnorm(q, qn, 1e-6), _ref_headnorm(k, kn, 1e-6)
    q, k = _ref_rope(q, pos, 1e6), _ref_rope(k, pos, 1e6)
    torch.testing.assert_close(q_out.float(), q, atol=3e-2, rtol=3e-2)
    flat_k, flat_v = kc.view(-1, hkv, d), vc.view(-1, hkv, d)
    keep = slots >= 0
    torch.testing.assert_close(flat_k[slots[keep].long()].float(), k[keep], atol=3e-2, rtol=3e-2)
    torch.testing.assert_close(flat_v[slots[keep].long()].float(), v[keep], atol=1e-6, rtol=0)
    assert int((flat_k.abs().sum((1, 2)) > 0).sum()) == int(keep.sum())


def _paged(batch, lens, hkv, d, page, device="cuda"):
    max_blocks = (max(lens) + page - 1) // page
    total = sum((l + page - 1) // page for l in lens) + 3
    perm = torch.randperm(total, device=device).int()
    table = torch.zeros(batch, max_blocks, dtype=torch.int32, device=device)
    c = 0
    for b, l in enumerate(lens):
        n = (l + page - 1) // page
        table[b, :n] = perm[c:c + n]
        c += n
    kc = torch.randn(total, page, hkv, d, device=device).bfloat16()
    vc = torch.randn(total, page, hkv, d, device=device).bfloat16()
    return kc, vc, table


def _gather(cache, table, b, n, page):
    idx = table[b, : (n + page - 1) // page].long()
    return cache[idx].reshape(-1, cache.shape[2], cache.shape[3])[:n].float()


@pytest.mark.parametrize("d,hq,hkv", [(128, 16, 8), (128, 32, 8), (128, 64, 8), (64, 4, 2), (128, 8, 8)])
@pytest.mark.parametrize("splits", [0, 1, 3])
@pytest.mark.parametrize("simt", [False, True])
def test_paged_decode(d, hq, hkv, splits, simt):
    from crosspool_b200.ops import attention as A

    torch.manual_seed(1)
    lens = [1, 15, 16, 17, 200, 1023, 64]
    page = 16
    kc, vc, table = _paged(len(lens), lens, hkv, d, page)
    q = torch.randn(len(lens), hq, d, device="cuda").bfloat16()
    sl = torch.tensor(lens, device="cuda", dtype=torch.int32)
    out = A.paged_decode(q, kc, vc, table, sl, num_splits=splits, force_simt=simt)
    g = hq // hkv
    for b, n in enumerate(lens):
        k, v = _gather(kc, table, b, n, page), _gather(vc, table, b, n, page)
        k, v = k.repeat_interleave(g, 1), v.repeat_interleave(g, 1)  # [n, hq, d]
        s = torch.einsum("hd,nhd->hn", q[b].float(), k) * d ** -0.5
        ref = torch.einsum("hn,nhd->hd", s.softmax(-1), v)
        torch.testing.assert_close(out[b].float(), ref, atol=2e-2, rtol=2e-2)


@pytest.mark.parametrize("d,hq,hkv", [(128, 16, 8), (64, 4, 2), (128, 32, 4), (128, 8, 8), (64, 8, 2)])
@pytest.mark.parametrize("simple,page", [(False, 16), (False, 64), ("umma-alt", 16), ("umma-alt", 64), (True, 16), ("mma", 16), ("mma", 64)])
def test_paged_prefill_chunked_causal(d, hq, hkv, simple, page):
    from crosspool_b200.ops import attention as A
    from crosspool_b200.ops import gemm

    torch.manual_seed(2)
    ctx = [0, 5, 128, 300, 0]
    qlen = [1, 70, 64, 130, 257]
    lens = [c + q for c, q in zip(ctx, qlen)]
    kc, vc, table = _paged(len(lens), lens, hkv, d, page)
    # slots past each sequence's end hold NaN (stale or unscrubbed memory): they must not leak into the result
    for b, n in enumerate(lens):
        if n % page:
            last = int(table[b, (n - 1) // page])
            kc[last, n % page:] = float("nan")
            vc[last, n % page:] = float("nan")
    total_q = sum(qlen)
    q = torch.randn(total_q, hq, d, device="cuda").bfloat16()
    starts = torch.tensor([sum(qlen[:i]) for i in range(len(qlen))], device="cuda", dtype=torch.int32)
    out = A.paged_prefill(q, kc, vc, table, starts, torch.tensor(qlen, device="cuda", dtype=torch.int32),
                          torch.tensor(ctx, device="cuda", dtype=torch.int32), max(qlen), force_simple=simple)
    torch.cuda.synchronize()
    gemm.check_status(q.device)
    assert torch.isfinite(out.float()).all()
    g = hq // hkv
    for b in range(len(lens)):
        n = lens[b]
        k, v = _gather(kc, table, b, n, page), _gather(vc, table, b, n, page)
        k, v = k.repeat_interleave(g, 1), v.repeat_interleave(g, 1)
        qb = q[int(starts[b]): int(starts[b]) + qlen[b]].float()
        s = torch.einsum("qhd,nhd->hqn", qb, k) * d ** -0.5
        qi = torch.arange(qlen[b], device="cuda")[:, None] + ctx[b]
        mask = torch.arange(n, device="cuda")[None, :] <= qi
        s = s.masked_fill(~mask[None], float("-inf"))
        ref = torch.einsum("hqn,nhd->qhd", s.softmax(-1), v)
        got = out[int(starts[b]): int(starts[b]) + qlen[b]].float()
        torch.testing.assert_close(got, ref, atol=2e-2, rtol=2e-2)


def test_embedding_and_argmax():
    from crosspool_b200.ops import attention as A

    torch.manual_seed(3)
    table = torch.randn(1000, 256, device="cuda").bfloat16()
    ids = torch.randint(0, 1000, (33,), device="cuda", dtype=torch.int32)
    assert torch.equal(A.embedding(ids, table), table[ids.long()])
    logits = torch.randn(9, 151936, device="cuda")
    logits[3, 77] = 100.0
    logits[3, 5000] = 100.0
    got = A.argmax(logits)
    assert torch.equal(got.long(), logits.argmax(-1))
    assert int(got[3]) == 77
    lb = logits.bfloat16()
    assert torch.equal(A.argmax(lb).long(), lb.float().argmax(-1))


@pytest.mark.parametrize("d,hq,hkv", [(128, 32, 2), (64, 16, 1)])
def test_tensor_core_decode_handles_sixteen_heads_per_group_and_ignores_stale_cache_slots(d, hq, hkv):
    from crosspool_b200.ops import attention as A
    from crosspool_b200.ops import gemm

    torch.manual_seed(7)
    lens = [5, 16, 37, 300, 513]
    page = 32
    kc, vc, table = _paged(len(lens), lens, hkv, d, page)
    # slots past each sequence's end hold NaN (as stale or unscrubbed memory might)
    for b, n in enumerate(lens):
        last = int(table[b, (n - 1) // page])
        kc[last, n % page or page:] = float("nan")
        vc[last, n % page or page:] = float("nan")
    q = torch.randn(len(lens), hq, d, device="cuda").bfloat16()
    sl = torch.tensor(lens, device="cuda", dtype=torch.int32)
    out = A.paged_decode(q, kc, vc, table, sl, num_splits=2, chunk_tokens=256)
    torch.cuda.synchronize()
    gemm.check_status(q.device)
    assert torch.isfinite(out.float()).all()
    g = hq // hkv
    for b, n in enumerate(lens):
        k, v = _gather(kc, table, b, n, page), _gather(vc, table, b, n, page)
        k, v = k.repeat_interleave(g, 1), v.repeat_interleave(g, 1)
        s = torch.einsum("hd,nhd->hn", q[b].float(), k) * d ** -0.5
        ref = torch.einsum("hn,nhd->hd", s.softmax(-1), v)
        torch.testing.assert_close(out[b].float(), ref, atol=2e-2, rtol=2e-2)


def test_paged_decode_fixed_chunks_balance_mixed_lengths():
    from crosspool_b200.ops import attention as A

    torch.manual_seed(4)
    d, hq, hkv, page = 128, 16, 8, 16
    lens = [1, 255, 256, 257, 700, 1500, 33] * 6
    kc, vc, table = _paged(len(lens), lens, hkv, d, page)
    q = torch.randn(len(lens), hq, d, device="cuda").bfloat16()
    sl = torch.tensor(lens, device="cuda", dtype=torch.int32)
    assert A.decode_plan(len(lens), hkv, 1520) == (2, 1024)      # 336 (sequence, head) pairs: two long slices
    assert A.decode_plan(256, hkv, 2048) == (1, 0) and A.decode_plan(4, hkv, 2048) == (8, 256)
    splits, chunk = 6, 256
    out = A.paged_decode(q, kc, vc, table, sl, num_splits=splits, chunk_tokens=chunk)
    ref = A.paged_decode(q, kc, vc, table, sl, num_splits=1)
    torch.testing.assert_close(out.float(), ref.float(), atol=1e-2, rtol=1e-2)


def test_gumbel_sampling_follows_the_softmax_and_is_reproducible():
    from crosspool_b200.ops import attention as A

    torch.manual_seed(11)
    rows, vocab = 4096, 1000
    base = torch.randn(vocab, device="cuda") * 2.0
    logits = base[None].repeat(rows, 1).bfloat16()
    temps = torch.full((rows,), 0.7, device="cuda")
    temps[:8] = 0.0                                           # greedy rows
    seeds = torch.stack([torch.arange(rows, device="cuda", dtype=torch.int32) + 17,
                         torch.zeros(rows, device="cuda", dtype=torch.int32)], dim=1).contiguous()
    tok = A.sample(logits, temps, seeds)
    assert torch.equal(tok[:8].long(), logits[:8].float().argmax(-1))
    assert torch.equal(tok, A.sample(logits, temps, seeds))   # same (seed, step) -> same token
    seeds2 = seeds.clone()
    seeds2[:, 1] = 1
    assert (A.sample(logits, temps, seeds2)[8:] != tok[8:]).float().mean() > 0.5   # next step draws anew
    p = (logits[0].float() / 0.7).softmax(-1)
    freq = torch.bincount(tok[8:].long(), minlength=vocab).float() / (rows - 8)
    top = p.topk(5).indices
    assert ((freq[top] - p[top]).abs() < 4 * (p[top] * (1 - p[top]) / (rows - 8)).sqrt() + 0.005).all()
    assert (freq - p).abs().sum().item() < 0.5                 # total variation distance well below a uniform draw's
