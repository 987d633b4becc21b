"""The allocation-free decode attention, called through its exported C symbol.

Some callers of this library may not allocate device memory at all (they run under a CUDA-graph capture,
or inside a host program that owns every byte of the GPU, or in a loop that cannot afford an allocation's
latency).  For them ``pih_paged_attention_mma_no_alloc`` keeps the kernel's scratch in a fixed array inside
the library.  This test calls it twice in a row — the second call finds the first call's leftovers in the
shared array — and checks both results against the ordinary entry point, which gets scratch from torch.
It also checks that a problem too large for the array is refused with a message.  The file sorts last so
that a run which stops at the first failure has already run every other test.
"""
import ctypes
import math

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
TOL = dict(rtol=1.6e-2, atol=4e-3)          # the tolerance of the tensor-core attention tests


def _problem(seed, lens, heads=16, kv_heads=8, D=128, page=16):
    g = torch.Generator().manual_seed(seed)
    R = len(lens)
    pages_per = [-(-n // page) for n in lens]
    num_pages = sum(pages_per) + 2
    perm = torch.randperm(num_pages, generator=g).tolist()
    table = torch.full((R, max(pages_per)), -1, dtype=torch.int32)
    for r, n in enumerate(pages_per):
        table[r, :n] = torch.tensor([perm.pop() for _ in range(n)], dtype=torch.int32)
    cache = torch.randn(num_pages, 2, kv_heads, page, D, generator=g).to(torch.bfloat16).to(DEV)
    q = torch.randn(R, (heads + 2 * kv_heads) * D, generator=g).to(torch.bfloat16).to(DEV)
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=DEV)
    from types import SimpleNamespace
    step = SimpleNamespace(num_requests=R, cu_q=i32(list(range(R + 1))), q_start=i32([n - 1 for n in lens]),
                           host_cu_q=list(range(R + 1)), host_q_start=[n - 1 for n in lens], attention_plans={},
                           request_of_row=i32(list(range(R))), positions=i32([n - 1 for n in lens]))
    return dict(q=q, cache=cache, table=table.to(DEV), step=step, lens=lens, heads=heads, kv_heads=kv_heads, D=D,
                page=page, num_pages=num_pages)


def _call_no_alloc(ops, p, split, message, claimed_ctx=None):
    lib = ops.lib
    fn = lib.pih_paged_attention_mma_no_alloc
    fn.restype = ctypes.c_int
    R = len(p["lens"])
    out = torch.zeros(R, p["heads"] * p["D"], dtype=torch.bfloat16, device=DEV)
    vp = lambda t: ctypes.c_void_p(0 if t is None else t.data_ptr())
    rc = fn(vp(p["q"]), p["q"].stride(0), vp(out), vp(p["cache"]), vp(p["table"]), p["table"].shape[1],
            vp(p["step"].cu_q), vp(p["step"].q_start), R, R, 0, 1, claimed_ctx or max(p["lens"]), p["heads"], p["kv_heads"], p["D"],
            p["page"], p["num_pages"], ctypes.c_float(1.0 / math.sqrt(p["D"])), 0, split,
            ops.kv_tensor_map(p["cache"]), vp(ops._error), ctypes.c_void_p(torch.cuda.current_stream().cuda_stream),
            message, len(message))
    return rc, out


def test_no_alloc_entry_point_matches_the_ordinary_one_twice_in_a_row():
    from pih_b200.kernels import get_ops
    ops = get_ops(torch.device(DEV))
    message = ctypes.create_string_buffer(256)
    split = 256
    for seed, lens in ((41, [2048, 77, 1000, 513]), (42, [300, 1999, 64, 1024])):     # two calls in a row
        p = _problem(seed, lens)
        ops.attention_split = split                 # the ordinary entry point with the same cut
        try:
            want = ops.paged_attention_mma(p["q"], heads=p["heads"], kv_heads=p["kv_heads"], head_dim=p["D"],
                                           kv_cache=p["cache"], block_table=p["table"], step=p["step"],
                                           scale=1.0 / math.sqrt(p["D"]), window=0)
        finally:
            ops.attention_split = 0
        rc, got = _call_no_alloc(ops, p, split, message)
        assert rc == 0, (rc, message.value)
        torch.cuda.synchronize()
        ops.check_errors()
        torch.testing.assert_close(got.float(), want.float(), **TOL)
        assert float(got.float().abs().max()) > 0.0


def test_no_alloc_entry_point_refuses_what_does_not_fit():
    from pih_b200.kernels import get_ops
    ops = get_ops(torch.device(DEV))
    message = ctypes.create_string_buffer(256)
    p = _problem(43, [100, 200])
    # a context of a million keys in splits of 64 would need hundreds of MB of partials: beyond the 8 MiB array
    rc, out = _call_no_alloc(ops, p, 64, message, claimed_ctx=1_000_000)
    assert rc == -3 and b"bytes of scratch" in message.value, (rc, message.value)
    torch.cuda.synchronize()
    assert float(out.float().abs().max()) == 0.0    # nothing was launched
