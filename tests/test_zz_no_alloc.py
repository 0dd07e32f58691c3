"""llmx_attn_decode_static: the decode-attention entry point for callers that cannot allocate device memory.

Some users of these kernels run where cudaMalloc is off limits when the kernel is called (inside another
framework's memory plan, in a plugin whose host owns the device's memory, in a loop that must not touch
the allocator).  For them the library exports one entry point whose workspace is a fixed array inside the
library itself.  This test calls it through its exported C symbol, twice in a row on different inputs
(the array keeps the first call's contents, which must not leak into the second), and holds its output to
the ordinary entry point's within the tolerance the attention tests use; it also checks that a request
beyond the array's stated size is refused.  The file sorts last so that a run that stops at the first
failure has already run every other test.
"""
import ctypes
import math

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

STATIC_FLOATS = 4 * 1024 * 1024      # LLMX_ATTN_DECODE_STATIC_FLOATS
TOO_LARGE = 10004


def _static_fn():
    from llmx_b200.csrc import build
    lib = build.load("attention_decode")
    fn = lib.llmx_attn_decode_static
    p, i, f = ctypes.c_void_p, ctypes.c_int, ctypes.c_float
    fn.argtypes = [p, p, p, p, i, p, p, p, p, i, i, i, i, i, i, i, f, i, i, i, p, p]
    fn.restype = ctypes.c_int
    return fn


def _call_static(fn, q, cache, step, group, heads, kv_heads, head_dim, splits, chunk):
    from llmx_b200 import ops_attn, ops_tc
    out = torch.full_like(q, float("nan"))
    cmap = ops_attn.cache_map(cache)
    n = step.requests
    req_list = torch.arange(n, dtype=torch.int32, device=q.device)
    status = fn(ctypes.c_void_p(cmap.address), q.data_ptr(), out.data_ptr(), req_list.data_ptr(), n,
                step.row_start.data_ptr(), step.row_count.data_ptr(), step.history.data_ptr(),
                group.block_tables.data_ptr(), group.block_tables.shape[1], q.shape[0], heads, kv_heads, head_dim,
                cache.shape[3], 0, 1.0 / math.sqrt(head_dim), splits, chunk, max(step.host_row_count),
                ops_tc.error_word(q.device).data_ptr(), torch.cuda.current_stream().cuda_stream)
    return status, out


def test_static_entry_point_matches_the_ordinary_one_on_two_calls_in_a_row():
    from llmx_b200 import ops_attn, ops_tc
    from test_kernels_gpu import _attention_case
    fn = _static_fn()
    heads, kv_heads, head_dim = 8, 2, 128
    layouts = ([(1500, 1), (63, 1), (700, 2), (0, 1)], [(90, 1), (2047, 1), (300, 1)])
    for call, layout in enumerate(layouts):
        q, cache, step, group, ref = _attention_case(torch.bfloat16, heads, kv_heads, head_dim, 16, layout, None,
                                                     seed=20 + call, spike=True)
        longest = max(h + n for h, n in layout)
        splits = 4
        chunk = -(-(-(-longest // 64)) // splits) * 64
        _req_list = torch.arange(step.requests, dtype=torch.int32, device=q.device)
        step.plan.native.plan.force_decode(splits, chunk)
        want = torch.full_like(q, float("nan"))
        ops_attn.paged_attention_bf16(q, cache, want, step, group, heads, kv_heads, head_dim, None, 1.0 / math.sqrt(head_dim))
        status, got = _call_static(fn, q, cache, step, group, heads, kv_heads, head_dim, splits, chunk)
        torch.cuda.synchronize()
        ops_tc.check_errors()
        assert status == 0
        if call == 1:
            # The set-up (the array's address) happened in the first call.  From here on a call must leave the
            # device's free memory exactly as it found it: were the entry point to allocate, even through a
            # pool, cudaMemGetInfo would show it.  Inputs and output exist already; only the call is repeated.
            out_again = torch.empty_like(q)
            cmap = ops_attn.cache_map(cache)          # held until the call returns: the launch reads the descriptor from host memory
            torch.cuda.synchronize()
            free_before, _ = torch.cuda.mem_get_info()
            reserved_before = torch.cuda.memory_reserved()
            status = fn(ctypes.c_void_p(cmap.address), q.data_ptr(), out_again.data_ptr(),
                        _req_list.data_ptr(), step.requests, step.row_start.data_ptr(), step.row_count.data_ptr(),
                        step.history.data_ptr(), group.block_tables.data_ptr(), group.block_tables.shape[1], q.shape[0],
                        heads, kv_heads, head_dim, cache.shape[3], 0, 1.0 / math.sqrt(head_dim), splits, chunk,
                        max(step.host_row_count), ops_tc.error_word(q.device).data_ptr(),
                        torch.cuda.current_stream().cuda_stream)
            torch.cuda.synchronize()
            assert status == 0
            assert torch.cuda.mem_get_info()[0] == free_before and torch.cuda.memory_reserved() == reserved_before
            assert torch.equal(out_again, got)
        got_np, want_np = got.float().cpu().numpy(), want.float().cpu().numpy()
        assert np.isfinite(got_np).all()
        scale = max(1.0, np.abs(ref).max())
        assert np.abs(got_np - want_np).max() <= 2e-2 * scale
        assert np.abs(got_np - ref).max() <= 2e-2 * scale


def test_static_entry_point_refuses_more_than_its_array_holds():
    from test_kernels_gpu import _attention_case
    fn = _static_fn()
    heads, kv_heads, head_dim = 8, 2, 128
    q, cache, step, group, _ = _attention_case(torch.bfloat16, heads, kv_heads, head_dim, 16, [(100, 1)], None, seed=30)
    # Claim so many rows that rows * heads * splits * (head_dim + 2) exceeds the array: refused before any launch.
    rows = STATIC_FLOATS // (heads * 4 * (head_dim + 2)) + 1
    out = torch.zeros_like(q)
    cmap_holder = []
    from llmx_b200 import ops_attn, ops_tc
    cmap = ops_attn.cache_map(cache)
    req_list = torch.zeros(1, dtype=torch.int32, device=q.device)
    status = fn(ctypes.c_void_p(cmap.address), q.data_ptr(), out.data_ptr(), req_list.data_ptr(), 1,
                step.row_start.data_ptr(), step.row_count.data_ptr(), step.history.data_ptr(),
                group.block_tables.data_ptr(), group.block_tables.shape[1], rows, heads, kv_heads, head_dim, 16, 0,
                0.1, 4, 64, 1, ops_tc.error_word(q.device).data_ptr(), torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    assert status == TOO_LARGE and not out.any()
