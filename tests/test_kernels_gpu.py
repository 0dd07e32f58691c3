"""Each kernel alone against a plain float32 reference of the same operation, at sizes other than the
engine's tiny models: ragged edges, widths that are no power of two, one row, many rows."""
import math

import numpy as np
import pytest
import torch

import plain_qwen3 as plain

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _bf16(t):
    return t.to(torch.bfloat16)


# ---------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("rows,width,vocab", [(1, 96, 50), (37, 100, 257), (300, 4096, 1000)])
def test_embed(dtype, rows, width, vocab):
    from llmx_b200 import ops
    g = torch.Generator().manual_seed(1)
    table = torch.randn(vocab, width, generator=g).to(dtype).to(DEV)
    ids = torch.randint(0, vocab, (rows,), generator=g, dtype=torch.int32).to(DEV)
    out = torch.empty(rows, width, dtype=torch.float32, device=DEV)
    ops.embed(table, ids, out)
    assert torch.equal(out, table.float()[ids.long()])


@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("rows,width,eps", [(1, 16, 1e-6), (33, 100, 1e-5), (7, 4096, 1e-6), (5, 5000, 1e-3)])
def test_rmsnorm(out_dtype, rows, width, eps):
    from llmx_b200 import ops
    g = torch.Generator().manual_seed(2)
    x = (torch.randn(rows, width, generator=g) * 3).to(DEV)
    w = (1 + 0.1 * torch.randn(width, generator=g)).to(DEV)
    out = torch.empty(rows, width, dtype=out_dtype, device=DEV)
    ops.rmsnorm(x, w, eps, out)
    ref = plain.rms_norm(x.cpu().numpy(), w.cpu().numpy(), eps)
    if out_dtype is torch.bfloat16:
        ref = plain.round_bf16(ref)
        assert np.abs(out.float().cpu().numpy() - ref).max() <= np.abs(ref).max() * 2 ** -7
    else:
        assert np.abs(out.cpu().numpy() - ref).max() <= 1e-5 * np.abs(ref).max()
    # Gathered rows: the head's pick of rows folded into the norm.
    idx = torch.tensor([rows - 1, 0], dtype=torch.int32, device=DEV)
    out2 = torch.empty(2, width, dtype=out_dtype, device=DEV)
    ops.rmsnorm(x, w, eps, out2, row_index=idx)
    assert torch.equal(out2, out[idx.long()])


@pytest.mark.parametrize("rows,width", [(1, 8), (19, 172), (64, 12288)])
def test_swiglu(rows, width):
    from llmx_b200 import ops
    g = torch.Generator().manual_seed(3)
    gu = (torch.randn(rows, 2 * width, generator=g) * 4).to(DEV)
    out = torch.empty(rows, width, dtype=torch.float32, device=DEV)
    ops.swiglu(gu, out)
    a = gu.cpu().numpy()
    ref = plain.silu(a[:, :width]) * a[:, width:]
    assert np.abs(out.cpu().numpy() - ref).max() <= 1e-5 * max(1.0, np.abs(ref).max())


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("heads,kv_heads,head_dim,rot,norm", [(4, 2, 16, 16, True), (6, 3, 32, 32, True), (3, 1, 48, 24, False),
                                                              (32, 8, 128, 128, True), (2, 2, 256, 64, True)])
@pytest.mark.parametrize("rows", [11, 70])
def test_head_norm_rope_kv(dtype, heads, kv_heads, head_dim, rot, norm, rows):
    """Per-head norm, rotation (whole or partial width) and the write into scattered cache slots
    (few rows and many: the kernel shares its work out differently)."""
    from llmx_b200 import ops
    page, pages = 8, 9
    g = torch.Generator().manual_seed(4)
    qkv = torch.randn(rows, (heads + 2 * kv_heads) * head_dim, generator=g).to(DEV)
    qw = (1 + 0.1 * torch.randn(head_dim, generator=g)).to(DEV) if norm else None
    kw = (1 + 0.1 * torch.randn(head_dim, generator=g)).to(DEV) if norm else None
    positions = torch.randint(0, 40, (rows,), generator=g, dtype=torch.int32)
    cos_np, sin_np = plain.rope_tables(40, rot, 10000.0)
    cos, sin = torch.from_numpy(cos_np).to(DEV), torch.from_numpy(sin_np).to(DEV)
    slots = torch.randperm(pages * page, generator=g)[:rows].to(torch.int32)
    slots[3] = -1                                                   # one row's write is skipped
    cache = torch.zeros(pages, 2, kv_heads, page, head_dim, dtype=dtype, device=DEV)
    q_out = torch.empty(rows, heads * head_dim, dtype=dtype, device=DEV)
    ops.head_norm_rope_kv(qkv, heads, kv_heads, head_dim, qw, kw, 1e-6, cos, sin, positions.to(DEV), slots.to(DEV),
                          q_out, cache)
    a = qkv.cpu().numpy()
    q = a[:, :heads * head_dim].reshape(rows, heads, head_dim)
    k = a[:, heads * head_dim:(heads + kv_heads) * head_dim].reshape(rows, kv_heads, head_dim)
    v = a[:, (heads + kv_heads) * head_dim:].reshape(rows, kv_heads, head_dim)
    if norm:
        q, k = plain.rms_norm(q, qw.cpu().numpy(), 1e-6), plain.rms_norm(k, kw.cpu().numpy(), 1e-6)
    c, s = cos_np[positions.numpy()], sin_np[positions.numpy()]

    def rotate(x):
        out = x.copy()
        out[..., :rot] = plain.rope_rotate(x[..., :rot], c, s)
        return out
    q, k = rotate(q), rotate(k)
    tol = 2 ** -7 if dtype is torch.bfloat16 else 1e-5
    got_q = q_out.float().cpu().numpy().reshape(rows, heads, head_dim)
    assert np.abs(got_q - q).max() <= tol * np.abs(q).max()
    cache_np = cache.float().cpu().numpy()
    for r in range(rows):
        sl = int(slots[r])
        if sl < 0:
            continue
        assert np.abs(cache_np[sl // page, 0, :, sl % page] - k[r]).max() <= tol * np.abs(k).max()
        assert np.abs(cache_np[sl // page, 1, :, sl % page] - v[r]).max() <= tol * np.abs(v).max()
    written = {int(s) for s in slots if s >= 0}
    for sl in range(pages * page):
        if sl not in written:
            assert not cache_np[sl // page, :, :, sl % page].any()


# ---------------------------------------------------------------------------------------------
@pytest.mark.parametrize("m,n,k", [(1, 64, 16), (5, 100, 37), (70, 257, 100), (130, 384, 96)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_gemm_plain(dtype, m, n, k):
    from llmx_b200 import ops
    g = torch.Generator().manual_seed(5)
    a = torch.randn(m, k, generator=g).to(dtype).to(DEV)
    w = torch.randn(n, k, generator=g).to(dtype).to(DEV)
    base = torch.randn(m, n, generator=g).to(DEV)
    ref = a.float().cpu().double() @ w.float().cpu().double().T
    out = torch.empty(m, n, dtype=torch.float32, device=DEV)
    ops.gemm_plain(a, w, out)
    assert (out.cpu().double() - ref).abs().max() <= 1e-5 * ref.abs().max()
    acc = base.clone()
    ops.gemm_plain(a, w, acc, accumulate=True)
    assert (acc.cpu().double() - (ref + base.cpu().double())).abs().max() <= 1e-5 * ref.abs().max()


@pytest.mark.parametrize("m", [1, 3, 16, 17, 64, 65, 128, 200, 513])
@pytest.mark.parametrize("n,k", [(128, 64), (100, 72), (384, 96), (1000, 160), (6144, 1024)])
def test_gemm_tensor_core(m, n, k):
    """The tcgen05 product at ragged sizes: M, N beyond a tile's edge, K that is no multiple of 64."""
    from llmx_b200 import ops_tc
    g = torch.Generator().manual_seed(6)
    a = _bf16(torch.randn(m, k, generator=g)).to(DEV)
    w = _bf16(torch.randn(n, k, generator=g) * 0.1).to(DEV)
    ref = a.float().cpu().double() @ w.float().cpu().double().T
    guard = torch.full((m + 2, n), 7.0, device=DEV)             # rows around the output must stay untouched
    out = guard[1:m + 1]
    ops_tc.gemm_tc(a, w, out)
    torch.cuda.synchronize()
    ops_tc.check_errors()
    assert (out.cpu().double() - ref).abs().max() <= 2e-5 * max(1.0, ref.abs().max())
    assert torch.all(guard[0] == 7.0) and torch.all(guard[m + 1] == 7.0)
    base = torch.randn(m, n, generator=g).to(DEV)
    for splits in (1, 2, 5):
        acc = base.clone()
        ops_tc.gemm_tc(a, w, acc, accumulate=True, splits=splits)
        assert (acc.cpu().double() - (ref + base.cpu().double())).abs().max() <= 3e-5 * max(1.0, ref.abs().max())
    ops_tc.check_errors()


@pytest.mark.parametrize("tile", [16, 32, 64, 128, 256])
def test_gemm_tensor_core_every_token_tile(tile):
    from llmx_b200 import ops_tc
    g = torch.Generator().manual_seed(7)
    m, n, k = 300, 260, 200
    a = _bf16(torch.randn(m, k, generator=g)).to(DEV)
    w = _bf16(torch.randn(n, k, generator=g)).to(DEV)
    out = torch.empty(m, n, device=DEV)
    ops_tc.gemm_tc(a, w, out, token_tile=tile)
    ref = a.float().cpu().double() @ w.float().cpu().double().T
    ops_tc.check_errors()
    assert (out.cpu().double() - ref).abs().max() <= 2e-5 * ref.abs().max()


@pytest.mark.parametrize("m", [65, 130, 257, 600])
@pytest.mark.parametrize("n,k", [(100, 72), (384, 96), (1000, 160), (4096, 1024)])
def test_gemm_tensor_core_on_pairs_of_sms(m, n, k):
    """The two-block (tcgen05 `cta_group::2`) product at ragged sizes: a second block whose weight rows or token rows
    lie wholly or partly beyond the matrix, K that is no multiple of 64, both token tiles, K in ranges."""
    from llmx_b200 import ops_tc
    g = torch.Generator().manual_seed(16)
    a = _bf16(torch.randn(m, k, generator=g)).to(DEV)
    w = _bf16(torch.randn(n, k, generator=g) * 0.1).to(DEV)
    ref = a.float().cpu().double() @ w.float().cpu().double().T
    base = torch.randn(m, n, generator=g).to(DEV)
    for tile in (128, 256):
        guard = torch.full((m + 2, n), 7.0, device=DEV)
        out = guard[1:m + 1]
        ops_tc.gemm_tc_pair(a, w, out, token_tile=tile)
        torch.cuda.synchronize()
        ops_tc.check_errors()
        assert (out.cpu().double() - ref).abs().max() <= 2e-5 * max(1.0, ref.abs().max())
        assert torch.all(guard[0] == 7.0) and torch.all(guard[m + 1] == 7.0)
        for splits in (1, 2, 3, 0):
            acc = base.clone()
            ops_tc.gemm_tc_pair(a, w, acc, accumulate=True, splits=splits, token_tile=tile)
            assert (acc.cpu().double() - (ref + base.cpu().double())).abs().max() <= 3e-5 * max(1.0, ref.abs().max())
    ops_tc.check_errors()


@pytest.mark.parametrize("m,n,k", [(2300, 2100, 1104), (1100, 4100, 3000), (520, 1000, 64), (4100, 2300, 8200)])
def test_gemm_on_pairs_cuts_only_the_last_round(m, n, k):
    """`splits` 0: whole tiles for the full rounds of the 74 pairs, the remaining tiles' K in ranges.  Sizes with one
    or two full rounds and a ragged rest, fewer tiles than pairs, a single k block, and a K long enough that the
    rest is cut into many ranges; added to what the output holds, and stored."""
    from llmx_b200 import ops_tc
    g = torch.Generator().manual_seed(18)
    a = _bf16(torch.randn(m, k, generator=g)).to(DEV)
    w = _bf16(torch.randn(n, k, generator=g) * 0.1).to(DEV)
    ref = a.float().double() @ w.float().double().T
    base = torch.randn(m, n, generator=g).to(DEV)
    bound = 3e-5 * max(1.0, ref.abs().max().item())
    for tile in (128, 256):
        acc = base.clone()
        ops_tc.gemm_tc_pair(a, w, acc, accumulate=True, splits=0, token_tile=tile)
        assert (acc.double() - (ref + base.double())).abs().max() <= bound
        guard = torch.full((m + 2, n), 7.0, device=DEV)
        out = guard[1:m + 1]
        ops_tc.gemm_tc_pair(a, w, out, splits=0, token_tile=tile)
        assert (out.double() - ref).abs().max() <= bound
        assert torch.all(guard[0] == 7.0) and torch.all(guard[m + 1] == 7.0)
    ops_tc.check_errors()


def test_gemm_plan_may_choose_pairs_and_can_be_told_not_to():
    from llmx_b200 import ops_tc, runtime
    assert ops_tc.plan(2048, 4096, 4096, True)[0] == 2
    before = runtime.pair_products(False)
    try:
        assert ops_tc.plan(2048, 4096, 4096, True)[0] == 0
    finally:
        runtime.pair_products(before)
    assert ops_tc.plan(8, 4096, 4096, True)[0] == 1


def test_gemm_tensor_core_refuses_unaligned_width():
    from llmx_b200 import ops_tc
    from llmx_b200.ops import KernelError
    a = torch.zeros(4, 100, dtype=torch.bfloat16, device=DEV)
    w = torch.zeros(8, 100, dtype=torch.bfloat16, device=DEV)
    with pytest.raises(KernelError):
        ops_tc.gemm_tc(a, w, torch.empty(4, 8, device=DEV))


# ---------------------------------------------------------------------------------------------
def _attention_case(dtype, heads, kv_heads, head_dim, page, layout, window, seed, spike=False):
    """A batch laid out as `layout` = [(history, new rows), ...] over a shuffled pool of pages.

    Returns everything the kernels need plus the plain result.  With `spike`, one far key of every
    request is made to stand out (its score dominates), so a kernel that drops or misplaces a page
    shows a large error instead of one that random values average away."""
    g = torch.Generator().manual_seed(seed)
    n_req = len(layout)
    lens = [h + n for h, n in layout]
    pages_needed = [-(-l // page) for l in lens]
    total_pages = sum(pages_needed) + 3
    perm = torch.randperm(total_pages, generator=g).tolist()
    cache = torch.randn(total_pages, 2, kv_heads, page, head_dim, generator=g)      # stale values everywhere
    tables = np.zeros((n_req, max(pages_needed)), dtype=np.int32)
    ks, vs, qs = [], [], []
    rows = sum(n for _, n in layout)
    row_start, at = [], 0
    for r, (h, n) in enumerate(layout):
        row_start.append(at)
        at += n
        k = torch.randn(lens[r], kv_heads, head_dim, generator=g)
        v = torch.randn(lens[r], kv_heads, head_dim, generator=g)
        q = torch.randn(n, heads, head_dim, generator=g)
        if spike and lens[r] > 3:
            far = max(0, lens[r] - (window or lens[r]) + 1) if window else 1
            far = min(far, lens[r] - 1)
            k[far] = q[-1, ::heads // kv_heads] * 4.0          # every group's key lines up with the last row's query
        ks.append(k); vs.append(v); qs.append(q)
        mine = [perm.pop() for _ in range(pages_needed[r])]
        tables[r, :len(mine)] = mine
        for t in range(lens[r]):
            cache[mine[t // page], 0, :, t % page] = k[t]
            cache[mine[t // page], 1, :, t % page] = v[t]
    cache = cache.to(dtype)
    q_all = torch.cat(qs).to(dtype)
    ref = np.zeros((rows, heads, head_dim), dtype=np.float32)
    for r, (h, n) in enumerate(layout):
        full_q = np.zeros((lens[r], heads, head_dim), dtype=np.float32)
        full_q[h:] = q_all[row_start[r]:row_start[r] + n].float().numpy()
        kk = ks[r].to(dtype).float().numpy()
        vv = vs[r].to(dtype).float().numpy()
        ref[row_start[r]:row_start[r] + n] = plain.attention(full_q, kk, vv, window=window)[h:]
    # The step (metadata on the device, launch plan of an attention of this shape) as the engine would make it.
    from llmx_b200 import ops_attn
    step = ops_attn.attention_step(DEV, layout, tables, heads, kv_heads, head_dim, window, page)
    group = step.groups[0]
    return q_all.reshape(rows, heads * head_dim).to(DEV).contiguous(), cache.to(DEV), step, group, ref.reshape(rows, -1)


LAYOUTS = {
    "decode": [(0, 1), (1, 1), (15, 1), (16, 1), (17, 1), (200, 1), (1027, 1)],
    "prefill": [(0, 1), (0, 2), (0, 17), (0, 130), (0, 300)],
    "mixed": [(40, 1), (0, 70), (128, 2), (63, 65), (5, 3), (300, 1), (16, 16)],
}


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("heads,kv_heads,head_dim,page", [(4, 2, 16, 8), (6, 3, 32, 16), (3, 1, 48, 4), (8, 8, 80, 16), (2, 1, 256, 32)])
@pytest.mark.parametrize("layout", ["decode", "prefill", "mixed"])
@pytest.mark.parametrize("window", [None, 19])
def test_attention_plain(dtype, heads, kv_heads, head_dim, page, layout, window):
    from llmx_b200 import ops
    q, cache, step, group, ref = _attention_case(dtype, heads, kv_heads, head_dim, page, LAYOUTS[layout], window, seed=8)
    out = torch.empty_like(q)
    ops.attention_plain(q, cache, out, step.row_request, step.positions, group.block_tables, heads, kv_heads, head_dim,
                        window, 1.0 / math.sqrt(head_dim))
    tol = 2e-2 if dtype is torch.bfloat16 else 2e-5
    assert np.abs(out.float().cpu().numpy() - ref).max() <= tol * max(1.0, np.abs(ref).max())


@pytest.mark.parametrize("heads,kv_heads,head_dim", [(32, 8, 128), (4, 4, 64), (16, 1, 128), (6, 2, 64), (8, 8, 128),
                                                     (40, 8, 128), (6, 2, 128), (12, 2, 128), (10, 2, 64), (7, 1, 128)])
@pytest.mark.parametrize("layout", ["decode", "prefill", "mixed"])
@pytest.mark.parametrize("window", [None, 100])
@pytest.mark.parametrize("spike", [False, True])
def test_attention_tiled_bf16(heads, kv_heads, head_dim, layout, window, spike):
    """The split-KV decode kernel and the tiled prefill kernel behind the one dispatch the mixer calls."""
    from llmx_b200 import ops_attn, ops_tc
    assert ops_attn.supported(heads, kv_heads, head_dim, 16)
    q, cache, step, group, ref = _attention_case(torch.bfloat16, heads, kv_heads, head_dim, 16, LAYOUTS[layout], window,
                                                 seed=9, spike=spike)
    out = torch.full_like(q, float("nan"))
    ops_attn.paged_attention_bf16(q, cache, out, step, group, heads, kv_heads, head_dim, window, 1.0 / math.sqrt(head_dim))
    torch.cuda.synchronize()
    ops_tc.check_errors()
    got = out.float().cpu().numpy()
    assert np.isfinite(got).all()
    assert np.abs(got - ref).max() <= 2e-2 * max(1.0, np.abs(ref).max())


@pytest.mark.parametrize("item_tiles,key_splits", [(1, 1), (2, 1), (1, 2), (2, 2), (2, 3), (1, 5)])
@pytest.mark.parametrize("heads,kv_heads", [(32, 8), (16, 8), (8, 8), (40, 8), (6, 2), (14, 2)])
@pytest.mark.parametrize("window", [None, 300])
def test_attention_prefill_items_of_any_shape(item_tiles, key_splits, heads, kv_heads, window):
    """The tcgen05 prefill kernel's work items hold one row tile or two, and all of a block's keys or one of
    several ranges of them (a second kernel then adds the ranges up); the launcher chooses, here every
    combination is forced.  Short requests leave ranges without keys and rows that a range's keys do not reach."""
    from llmx_b200 import ops_attn, ops_tc
    layout = [(0, 300), (77, 130), (1500, 64), (3, 33), (40, 1), (700, 200)]
    q, cache, step, group, ref = _attention_case(torch.bfloat16, heads, kv_heads, 128, 16, layout, window, seed=23, spike=True)
    step.plan.native.plan.force_prefill_shape(item_tiles, key_splits)
    out = torch.full_like(q, float("nan"))
    ops_attn.paged_attention_bf16(q, cache, out, step, group, heads, kv_heads, 128, window, 1.0 / math.sqrt(128))
    torch.cuda.synchronize()
    ops_tc.check_errors()
    got = out.float().cpu().numpy()
    assert np.isfinite(got).all()
    assert np.abs(got - ref).max() <= 2e-2 * max(1.0, np.abs(ref).max())


@pytest.mark.parametrize("history", [0, 320, 448])
def test_attention_prefill_blocks_walk_several_items(history):
    """More work items than SMs: a block of the tcgen05 prefill kernel then walks several (request, kv head, rows)
    items one after the other, its barriers' phases going on from item to item.  Forty requests of 64 new rows
    after the same history make 320 items of equal length, which is what once let a barrier complete twice
    before a waiting warp had looked."""
    from llmx_b200 import ops_attn, ops_tc
    heads, kv_heads, head_dim = 32, 8, 128
    layout = [(history, 64)] * 38 + [(history + 100, 33), (7, 130)]
    q, cache, step, group, ref = _attention_case(torch.bfloat16, heads, kv_heads, head_dim, 16, layout, None, seed=21, spike=True)
    for _ in range(3):                                   # the fault was one of timing: run it more than once
        out = torch.full_like(q, float("nan"))
        ops_attn.paged_attention_bf16(q, cache, out, step, group, heads, kv_heads, head_dim, None, 1.0 / math.sqrt(head_dim))
        torch.cuda.synchronize()
        ops_tc.check_errors()
        got = out.float().cpu().numpy()
        assert np.isfinite(got).all()
        assert np.abs(got - ref).max() <= 2e-2 * max(1.0, np.abs(ref).max())


@pytest.mark.parametrize("window", [None, 5000])
def test_attention_over_long_histories(window):
    """Tens of thousands of keys behind a request: block tables of over a thousand pages, sixteen key ranges for the
    decoding rows, hundreds of key stages for a prompt portion.  One key near the start of every request (or of
    its window) is made to stand out for the last row, so a page that is dropped or misplaced anywhere shows."""
    from llmx_b200 import ops_attn, ops_tc
    heads, kv_heads, D, page = 32, 8, 128, 16
    layout = [(20000, 1), (9001, 3), (12345, 70), (33, 1)]
    g = torch.Generator().manual_seed(31)
    lens = [h + n for h, n in layout]
    pages_needed = [-(-l // page) for l in lens]
    total_pages = sum(pages_needed) + 5
    perm = torch.randperm(total_pages, generator=g).tolist()
    cache = torch.randn(total_pages, 2, kv_heads, page, D, generator=g).to(torch.bfloat16)
    tables = np.zeros((len(layout), max(pages_needed)), dtype=np.int32)
    qs, refs, row_start, at = [], [], [], 0
    for r, (h, n) in enumerate(layout):
        row_start.append(at)
        at += n
        k = torch.randn(lens[r], kv_heads, D, generator=g)
        v = torch.randn(lens[r], kv_heads, D, generator=g)
        q = torch.randn(n, heads, D, generator=g).to(torch.bfloat16)
        far = max(1, lens[r] - window + 1) if window else 1
        k[far] = q[-1, ::heads // kv_heads].float() * 4.0
        k, v = k.to(torch.bfloat16), v.to(torch.bfloat16)
        mine = [perm.pop() for _ in range(pages_needed[r])]
        tables[r, :len(mine)] = mine
        idx = torch.tensor(mine).repeat_interleave(page)[:lens[r]]
        off = torch.arange(lens[r]) % page
        cache[idx, 0, :, off] = k
        cache[idx, 1, :, off] = v
        # plain reference for the new rows alone: row at position p sees keys lo..p
        kk = k.double().repeat_interleave(heads // kv_heads, dim=1)      # [L, heads, D]
        vv = v.double().repeat_interleave(heads // kv_heads, dim=1)
        scores = torch.einsum("nhd,lhd->nhl", q.double(), kk) / math.sqrt(D)
        pos = torch.arange(h, h + n)[:, None, None]
        keys = torch.arange(lens[r])[None, None, :]
        seen = keys <= pos
        if window:
            seen &= keys > pos - window
        scores = scores.masked_fill(~seen, float("-inf"))
        refs.append(torch.einsum("nhl,lhd->nhd", torch.softmax(scores, dim=-1), vv))
        qs.append(q)
    rows = at
    ref = torch.cat(refs).reshape(rows, -1).numpy()
    q_all = torch.cat(qs).reshape(rows, heads * D).to(DEV).contiguous()

    step = ops_attn.attention_step(DEV, layout, tables, heads, kv_heads, D, window, page)
    group = step.groups[0]
    out = torch.full_like(q_all, float("nan"))
    ops_attn.paged_attention_bf16(q_all, cache.to(DEV), out, step, group, heads, kv_heads, D, window, 1.0 / math.sqrt(D))
    torch.cuda.synchronize()
    ops_tc.check_errors()
    got = out.float().cpu().numpy()
    assert np.isfinite(got).all()
    assert np.abs(got - ref).max() <= 2e-2 * max(1.0, np.abs(ref).max())


@pytest.mark.parametrize("cluster", [True, False])
@pytest.mark.parametrize("splits", [1, 2, 3, 4, 7, 8, 12, 16, 20])
def test_attention_decode_any_number_of_key_ranges(splits, cluster):
    """Key ranges are combined through the shared memory of a thread-block cluster (up to sixteen ranges, unless
    turned off) or through memory by the block that finishes last; short requests leave ranges without keys."""
    from llmx_b200 import ops_attn, ops_tc
    before = ops_attn.cluster_merge(cluster)
    try:
        _decode_with_key_ranges(splits)
    finally:
        ops_attn.cluster_merge(before)


def _decode_with_key_ranges(splits):
    from llmx_b200 import ops_attn, ops_tc
    heads, kv_heads, head_dim = 8, 2, 128
    layout = [(1500, 1), (63, 1), (64, 1), (700, 2), (0, 1)]
    q, cache, step, group, ref = _attention_case(torch.bfloat16, heads, kv_heads, head_dim, 16, layout, None, seed=10, spike=True)
    chunk = -(-(-(-1501 // 64)) // splits) * 64
    step.plan.native.plan.force_decode(splits, chunk)
    out = torch.full_like(q, float("nan"))
    ops_attn.paged_attention_bf16(q, cache, out, step, group, heads, kv_heads, head_dim, None, 1.0 / math.sqrt(head_dim))
    torch.cuda.synchronize()
    ops_tc.check_errors()
    assert np.abs(out.float().cpu().numpy() - ref).max() <= 2e-2 * max(1.0, np.abs(ref).max())


@pytest.mark.parametrize("heads,kv_heads", [(32, 8), (16, 1), (8, 8), (4, 2)])
@pytest.mark.parametrize("window", [None, 100])
@pytest.mark.parametrize("rotate,norm", [(True, True), (False, True), (True, False)])
@pytest.mark.parametrize("splits", [None, 3])
def test_attention_decode_from_the_products_output(heads, kv_heads, window, rotate, norm, splits):
    """The decode kernel that norms and rotates its own queries and new keys, against the separate kernel
    followed by the decode kernel: the same bits in the output and in the cache.  Histories put new rows at
    the first and last slot of a page, at the edge of a key range, and (with several new rows) across two pages;
    one request's write is skipped, as for a layer that reads another layer's cache."""
    from llmx_b200 import ops, ops_attn, ops_tc
    head_dim, page = 128, 16
    max_new = 16 // (heads // kv_heads)
    layout = [(0, 1), (15, 1), (16, 1), (63, min(2, max_new)), (64, 1), (127, min(3, max_new)), (700, max_new), (1500, 1)]
    _, cache, step, group, _ = _attention_case(torch.bfloat16, heads, kv_heads, head_dim, page, layout, window, seed=12)
    rows = step.rows
    g = torch.Generator().manual_seed(13)
    qkv = torch.randn(rows, (heads + 2 * kv_heads) * head_dim, generator=g).to(DEV)
    qw = (1 + 0.1 * torch.randn(head_dim, generator=g)).to(DEV) if norm else None
    kw = (1 + 0.1 * torch.randn(head_dim, generator=g)).to(DEV) if norm else None
    cos = sin = None
    if rotate:
        cos_np, sin_np = plain.rope_tables(1600, head_dim, 10000.0)
        cos, sin = torch.from_numpy(cos_np).to(DEV), torch.from_numpy(sin_np).to(DEV)
    slots = group.slots                                             # page * 16 + slot of every row's position
    slots[step.host_row_start[4]] = -1                              # this row's key and value are not written
    if splits:
        step.plan.native.plan.force_decode(splits, -(-(-(-1501 // 64)) // splits) * 64)
    scale = 1.0 / math.sqrt(head_dim)
    # the separate kernels
    cache_a = cache.clone()
    q = torch.empty(rows, heads * head_dim, dtype=torch.bfloat16, device=DEV)
    ops.head_norm_rope_kv(qkv, heads, kv_heads, head_dim, qw, kw, 1e-6, cos, sin, step.positions, slots, q, cache_a)
    out_a = torch.full_like(q, float("nan"))
    ops_attn.paged_attention_bf16(q, cache_a, out_a, step, group, heads, kv_heads, head_dim, window, scale)
    # the one kernel
    cache_b = cache.clone()
    out_b = torch.full_like(q, float("nan"))
    assert ops_attn.decode_from_qkv(qkv, qw, kw, 1e-6, cos, sin, out_b, step, 0, heads, kv_heads, head_dim, window, scale,
                                    cache=ops_attn.OneEntryCache(cache_b))
    torch.cuda.synchronize()
    ops_tc.check_errors()
    assert torch.isfinite(out_b.float()).all()
    assert torch.equal(cache_a, cache_b)
    assert torch.equal(out_a, out_b)


# ---------------------------------------------------------------------------------------------
def _sample_rows(logits, settings):
    from llmx_b200.sampling import RequestSampling, SamplingParams, sample
    states = []
    for s in settings:
        st = RequestSampling(SamplingParams(**{k: v for k, v in s.items() if k not in ("gen", "masked")}),
                             eos_id=s.get("masked", -1))
        st.masked = s.get("masked", -1)
        for t in s.get("gen", ()):
            st.saw(t)
        states.append(st)
    got = sample(torch.from_numpy(logits).to(DEV).contiguous(), states)
    return got, states


@pytest.mark.parametrize("vocab", [5, 257, 5000, 151936])
def test_sampling_against_the_plain_sampler(vocab):
    """Every mode of the device sampler against the plain one, the same uniform number for both."""
    rng = np.random.default_rng(vocab)
    settings = [
        dict(temp=0.0, top_k=0, top_p=1.0),
        dict(temp=0.0, top_k=0, top_p=1.0, masked=0),
        dict(temp=1.0, top_k=0, top_p=1.0, seed=3),
        dict(temp=0.7, top_k=40, top_p=1.0, seed=4),
        dict(temp=1.3, top_k=0, top_p=0.9, seed=5),
        dict(temp=0.8, top_k=40, top_p=0.95, seed=6),
        dict(temp=1.0, top_k=3, top_p=0.5, min_p=0.2, seed=7),
        dict(temp=2.0, top_k=0, top_p=1.0, min_p=0.05, seed=8),
        dict(temp=1.0, top_k=0, top_p=0.8, min_p=0.1, seed=9, masked=1),
        dict(temp=0.0, top_k=0, top_p=1.0, penalty=1.5, presence_penalty=0.2, frequency_penalty=0.1, gen=[1, 2, 2, 4]),
        dict(temp=0.9, top_k=10, top_p=0.9, penalty=1.2, seed=11, gen=[0, 3]),
    ]
    logits = (rng.standard_normal((len(settings), vocab)) * 3).astype(np.float32)
    logits[0, :] = 0.0
    logits[0, [2, 4]] = 5.0                                  # a tie: the lowest id wins
    logits[3, :min(vocab, 60)] = 2.0                         # ties across the top-k edge: lowest ids are kept
    expected = []
    for row, s in zip(logits, settings):
        r = 0.0 if s["temp"] <= 0 else plain.XorShift64(s.get("seed", 0)).unit()
        expected.append(plain.sample(row, s["temp"], s["top_k"], s["top_p"], s.get("min_p", 0.0), r,
                                     penalty=s.get("penalty", 1.0), presence=s.get("presence_penalty", 0.0),
                                     frequency=s.get("frequency_penalty", 0.0), gen=list(s.get("gen", ())),
                                     masked=s.get("masked", -1)))
    got, _ = _sample_rows(logits.copy(), settings)
    assert got == expected


@pytest.mark.parametrize("vocab", [9001, 40000, 151936])
@pytest.mark.parametrize("coarse", [False, True])
def test_sampling_settings_at_random_against_the_plain_sampler(vocab, coarse):
    """Vocabularies that two, four and eight blocks share (see the end); settings drawn at random (top-k beyond what is gathered into
    shared memory too); with `coarse`, scores on a grid of quarters, so that hundreds of tokens tie exactly at every
    threshold: ties go to the lowest ids, whichever block holds them."""
    rng = np.random.default_rng(vocab + int(coarse))
    settings = []
    for i in range(24):
        settings.append(dict(temp=float(rng.choice([0.3, 0.8, 1.0, 1.7])), top_k=int(rng.choice([0, 1, 7, 40, 300, 1024, 1025, 3000])),
                             top_p=float(rng.choice([1.0, 0.95, 0.6, 0.1])), min_p=float(rng.choice([0.0, 0.0, 0.05, 0.3])),
                             seed=int(rng.integers(1, 1 << 40))))
        if i % 5 == 0:
            settings[-1]["masked"] = int(rng.integers(0, vocab))
    logits = (rng.standard_normal((len(settings), vocab)) * 2.5).astype(np.float32)
    if coarse:
        logits = (np.round(logits * 4) / 4).astype(np.float32)
    expected = []
    for row, s in zip(logits, settings):
        r = plain.XorShift64(s["seed"]).unit()
        expected.append(plain.sample(row, s["temp"], s["top_k"], s["top_p"], s["min_p"], r, masked=s.get("masked", -1)))
    got, _ = _sample_rows(logits.copy(), settings)
    assert got == expected
    # The kernel gives a row fewer blocks when the rows are many (all rows run at one time): twelve rows a call still
    # get the most blocks their vocabulary allows, twenty-four at the largest vocabulary get half as many.
    halves = _sample_rows(logits[:12].copy(), settings[:12])[0] + _sample_rows(logits[12:].copy(), settings[12:])[0]
    assert halves == expected


def test_sampling_distribution_and_independence_of_the_batch():
    """Draws follow the softmax, and a request's draws do not depend on what shares its batch."""
    from llmx_b200.sampling import RequestSampling, SamplingParams, sample
    logits = torch.tensor([[0.0, 1.0, 2.0, -1.0]], device=DEV)
    st = RequestSampling(SamplingParams(temp=1.0, top_k=0, top_p=1.0, seed=99))
    counts = np.zeros(4)
    alone = []
    for _ in range(2000):
        t = sample(logits, [st])[0]
        alone.append(t)
        counts[t] += 1
    p = np.exp([0, 1, 2, -1.0]); p /= p.sum()
    assert np.abs(counts / counts.sum() - p).max() < 0.04
    st2 = RequestSampling(SamplingParams(temp=1.0, top_k=0, top_p=1.0, seed=99))
    other = RequestSampling(SamplingParams(temp=0.5, top_k=2, top_p=0.9, seed=5))
    both = torch.cat([torch.randn(1, 4, device=DEV), logits])
    batched = [sample(both, [other, st2])[1] for _ in range(200)]
    assert batched == alone[:200]


@pytest.mark.parametrize("m", [1, 8, 33, 64])
@pytest.mark.parametrize("n,k", [(128, 64), (100, 72), (1000, 160), (6144, 1024), (4096, 4096), (5000, 4104)])
def test_gemm_tensor_core_stream_k(m, n, k):
    """Few tokens: (tile, k block) units shared out over the blocks, pieces added with atomics.  The two largest
    weights stream long enough to get uneven shares (the second half of the blocks a shorter run each)."""
    from llmx_b200 import ops_tc
    g = torch.Generator().manual_seed(12)
    a = _bf16(torch.randn(m, k, generator=g)).to(DEV)
    w = _bf16(torch.randn(n, k, generator=g) * 0.1).to(DEV)
    ref = a.float().cpu().double() @ w.float().cpu().double().T
    out = torch.full((m, n), 5.0, device=DEV)
    ops_tc.gemm_tc(a, w, out, schedule=1)
    assert (out.cpu().double() - ref).abs().max() <= 3e-5 * max(1.0, ref.abs().max())
    base = torch.randn(m, n, generator=g).to(DEV)
    acc = base.clone()
    ops_tc.gemm_tc(a, w, acc, accumulate=True, schedule=1)
    ops_tc.check_errors()
    assert (acc.cpu().double() - (ref + base.cpu().double())).abs().max() <= 3e-5 * max(1.0, ref.abs().max())


@pytest.mark.parametrize("pair", [False, True])
@pytest.mark.parametrize("m", [1, 16, 70, 128, 300])
@pytest.mark.parametrize("f,k", [(128, 64), (172, 104), (200, 128), (1536, 512)])
def test_gemm_tensor_core_gated(m, f, k, pair):
    """silu(gate) * up in the product's epilogue, for intermediate widths that are no multiple of a tile; on single
    blocks and on pairs of SMs."""
    from llmx_b200 import ops_tc
    g = torch.Generator().manual_seed(13)
    a = _bf16(torch.randn(m, k, generator=g)).to(DEV)
    w = _bf16(torch.randn(2 * f, k, generator=g) * 0.2).to(DEV)
    guard = torch.full((m + 2, f), 3.0, dtype=torch.bfloat16, device=DEV)
    out = guard[1:m + 1]
    ops_tc.gemm_tc_swiglu(a, w, out, pair=pair)
    ops_tc.check_errors()
    assert torch.all(guard[0] == 3.0) and torch.all(guard[m + 1] == 3.0)
    gu = (a.float().cpu().double() @ w.float().cpu().double().T).numpy()
    ref = plain.silu(gu[:, :f].astype(np.float32)) * gu[:, f:].astype(np.float32)
    assert np.abs(out.float().cpu().numpy() - ref).max() <= 2 ** -7 * max(1.0, np.abs(ref).max())


@pytest.mark.parametrize("tile", [128, 256, "pair"])
@pytest.mark.parametrize("m,heads,kv_heads,k,rotate,norm", [(70, 4, 2, 64, True, True), (300, 3, 1, 200, True, True),
                                                            (129, 2, 2, 512, False, True), (1000, 5, 1, 136, True, False)])
def test_gemm_tensor_core_finishes_heads(tile, m, heads, kv_heads, k, rotate, norm):
    """The q/k/v product with the per-head norm, the rotation and the cache write in its epilogue: against the
    plain formulas, and bit for bit against the product followed by the per-head kernel (a prompt's keys must
    not depend on which of the two a portion's size chose).  Odd head counts leave half-empty 256-row tiles."""
    from llmx_b200 import ops, ops_tc
    D, page, pages = 128, 16, 80
    g = torch.Generator().manual_seed(21)
    a = _bf16(torch.randn(m, k, generator=g)).to(DEV)
    w = _bf16(torch.randn((heads + 2 * kv_heads) * D, k, generator=g) * 0.2).to(DEV)
    qw = (1 + 0.1 * torch.randn(D, generator=g)).to(DEV) if norm else None
    kw = (1 + 0.1 * torch.randn(D, generator=g)).to(DEV) if norm else None
    positions = torch.randint(0, 300, (m,), generator=g, dtype=torch.int32)
    cos_np, sin_np = plain.rope_tables(300, D, 10000.0)
    cos = torch.from_numpy(cos_np).to(DEV) if rotate else None
    sin = torch.from_numpy(sin_np).to(DEV) if rotate else None
    slots = torch.randperm(pages * page, generator=g)[:m].to(torch.int32)
    slots[5] = -1
    cache = torch.zeros(pages, 2, kv_heads, page, D, dtype=torch.bfloat16, device=DEV)
    q_out = torch.zeros(m, heads * D, dtype=torch.bfloat16, device=DEV)
    pair = tile == "pair"       # on pairs of SMs: 256 tokens x two heads a pair, each block loads one head
    ops_tc.gemm_tc_heads(a, ops_tc.WeightMap(w, 128 if pair else tile, heads=True), heads, kv_heads, qw, kw, 1e-6, cos, sin,
                         positions.to(DEV), slots.to(DEV), q_out, cache, pair=pair)
    ops_tc.check_errors()

    qkv = torch.empty(m, w.shape[0], device=DEV)
    ops_tc.gemm_tc(a, w, qkv, schedule=0, splits=1)
    cache2, q2 = torch.zeros_like(cache), torch.zeros_like(q_out)
    ops.head_norm_rope_kv(qkv, heads, kv_heads, D, qw, kw, 1e-6, cos, sin, positions.to(DEV), slots.to(DEV), q2, cache2)
    assert torch.equal(q_out, q2) and torch.equal(cache, cache2)

    full = (a.float().cpu().double() @ w.float().cpu().double().T).numpy().astype(np.float32)
    q = full[:, :heads * D].reshape(m, heads, D)
    kk = full[:, heads * D:(heads + kv_heads) * D].reshape(m, kv_heads, D)
    v = full[:, (heads + kv_heads) * D:].reshape(m, kv_heads, D)
    if norm:
        q, kk = plain.rms_norm(q, qw.cpu().numpy(), 1e-6), plain.rms_norm(kk, kw.cpu().numpy(), 1e-6)
    if rotate:
        c, s = cos_np[positions.numpy()], sin_np[positions.numpy()]
        q, kk = plain.rope_rotate(q, c, s), plain.rope_rotate(kk, c, s)
    tol = 2 ** -7
    assert np.abs(q_out.float().cpu().numpy().reshape(m, heads, D) - q).max() <= tol * np.abs(q).max()
    cache_np = cache.float().cpu().numpy()
    for r in range(m):
        sl = int(slots[r])
        if sl >= 0:
            assert np.abs(cache_np[sl // page, 0, :, sl % page] - kk[r]).max() <= tol * np.abs(kk).max()
            assert np.abs(cache_np[sl // page, 1, :, sl % page] - v[r]).max() <= tol * np.abs(v).max()


def test_a_wait_that_nothing_satisfies_gives_up_and_is_reported():
    """Every wait in the kernels is bounded; a wait that runs out records a code in the device's error word and the
    block goes on to its end.  The self-test kernel (csrc/selftest.cu) waits a millisecond on a barrier nobody
    arrives at: the kernel returns, the word holds the code, and `check_errors` raises (and clears the word)."""
    import ctypes
    from llmx_b200 import ops_tc, runtime
    from llmx_b200.csrc import build
    fn = build.load("selftest").llmx_wait_selftest
    fn.argtypes = [ctypes.c_ulonglong, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p]
    fn.restype = ctypes.c_int
    torch.cuda.synchronize()
    ops_tc.check_errors()
    word = runtime.error_word(DEV)
    out = torch.zeros(2, dtype=torch.int32, device=DEV)
    assert fn(1_000_000, word.data_ptr(), out.data_ptr(), torch.cuda.current_stream().cuda_stream) == 0
    torch.cuda.synchronize()                                    # returns: nothing hangs
    assert out.tolist() == [2, 2]                               # the wait gave up; a later wait of the block returned at once
    with pytest.raises(runtime.KernelError, match="nobody arrives"):
        ops_tc.check_errors()
    ops_tc.check_errors()                                       # the word was cleared
    assert fn(10, word.data_ptr(), out.data_ptr(), None) == 10001          # limits outside 1 us .. 0.1 s are refused


def test_random_weights_are_the_same_on_the_device_and_on_the_host():
    """"Seed 0" names one model: the random-weights mode makes the same bits on the GPU (benchmarks, `Engine.from_config`)
    as on the CPU (model folders, the tests' plain implementation)."""
    from llmx_b200.weights.random_init import RandomSource
    from llmx_b200.weights.spec import TensorSpec
    specs = {"w.weight": TensorSpec((301, 257)), "n.weight": TensorSpec((129,), "vector", init="one_plus_normal", std=0.01)}
    for dtype in (torch.float32, torch.bfloat16):
        host, device = RandomSource(specs, 7, dtype=dtype, device="cpu"), RandomSource(specs, 7, dtype=dtype, device=DEV)
        for name in specs:
            assert torch.equal(host.tensor(name), device.tensor(name).cpu()), (name, dtype)
