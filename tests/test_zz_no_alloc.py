"""The allocation-free decode attention, called through its exported C symbol.

Some callers of this library may not allocate device memory at all: they are a plugin of a host program that
owns every byte of the GPU, they run after a set-up phase whose end freezes the process's allocations, or they
sit in a loop that cannot afford an allocation's latency or its failure.  For them
``pih_paged_attention_mma_no_alloc`` keeps the kernel's scratch — tickets and per-split partial results — in a
fixed array inside the library.

The calls here are cut so finely (more than eight splits a request, or the cluster merge switched off) that
the splits really merge through that array.  They run back to back: a large problem first, then, after the
whole array has been overwritten with junk (tickets that are not zero, partials that are NaN), a smaller one
that finds the junk, then one that needs nearly all of the 8 MiB.  Each result is checked against the plain
implementation's attention in float64, not against another path of the engine.  A problem too large for the
array must be refused with a message and launch nothing.  The file sorts last so that a run which stops at the
first failure has already run every other test.
"""
import ctypes
import math

import pytest
import torch

import plain_impl

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
TOL = dict(rtol=1.6e-2, atol=4e-3)          # the tolerance of the tensor-core attention tests
SCRATCH_BYTES = 8 * 1024 * 1024


def _problem(seed, lens, heads=16, kv_heads=8, D=128, page=16):
    g = torch.Generator().manual_seed(seed)
    R = len(lens)
    pages_per = [-(-n // page) for n in lens]
    num_pages = sum(pages_per) + 2
    perm = torch.randperm(num_pages, generator=g).tolist()
    table = torch.full((R, max(pages_per)), -1, dtype=torch.int32)
    for r, n in enumerate(pages_per):
        table[r, :n] = torch.tensor([perm.pop() for _ in range(n)], dtype=torch.int32)
    cache = torch.randn(num_pages, 2, kv_heads, page, D, generator=g).to(torch.bfloat16)
    q = torch.randn(R, (heads + 2 * kv_heads) * D, generator=g).to(torch.bfloat16)
    # the plain implementation's answer: each request's one query row over its own keys, in float64
    want = []
    for r, n in enumerate(lens):
        pages = table[r, :pages_per[r]].long()
        k = cache[pages, 0].permute(0, 2, 1, 3).reshape(-1, kv_heads, D)[:n]
        v = cache[pages, 1].permute(0, 2, 1, 3).reshape(-1, kv_heads, D)[:n]
        want.append(plain_impl.attention_rows(q[r, :heads * D].reshape(1, heads, D), [n - 1], k, v,
                                              1.0 / math.sqrt(D)).reshape(1, heads * D))
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=DEV)
    return dict(q=q.to(DEV), cache=cache.to(DEV), table=table.to(DEV), cu_q=i32(list(range(R + 1))),
                q_start=i32([n - 1 for n in lens]), want=torch.cat(want), lens=lens, heads=heads, kv_heads=kv_heads,
                D=D, page=page, num_pages=num_pages)


def _call_no_alloc(ops, p, split, message, claimed_ctx=None):
    fn = ops.lib.pih_paged_attention_mma_no_alloc
    fn.restype = ctypes.c_int
    R = len(p["lens"])
    out = torch.zeros(R, p["heads"] * p["D"], dtype=torch.bfloat16, device=DEV)
    vp = lambda t: ctypes.c_void_p(0 if t is None else t.data_ptr())
    rc = fn(vp(p["q"]), p["q"].stride(0), vp(out), vp(p["cache"]), vp(p["table"]), p["table"].shape[1],
            vp(p["cu_q"]), vp(p["q_start"]), R, R, 0, 1, claimed_ctx or max(p["lens"]), p["heads"], p["kv_heads"], p["D"],
            p["page"], p["num_pages"], ctypes.c_float(1.0 / math.sqrt(p["D"])), 0, split,
            ops.kv_tensor_map(p["cache"]), vp(ops.error_word), ctypes.c_void_p(torch.cuda.current_stream().cuda_stream),
            message, len(message))
    return rc, out


def _scratch_need(ops, p, split):
    ops.lib.pih_attention_scratch_floats.restype = ctypes.c_longlong
    return 4 * ops.lib.pih_attention_scratch_floats(len(p["lens"]), 1, p["heads"], p["kv_heads"], p["D"],
                                                    -(-max(p["lens"]) // split))


class _Array:
    """The library's array as torch sees a foreign device buffer."""

    def __init__(self, address, words):
        self.__cuda_array_interface__ = {"shape": (words,), "typestr": "<i4", "data": (address, False), "version": 2}


def _library_scratch(ops):
    ops.lib.pih_no_alloc_scratch_address.restype = ctypes.c_void_p
    address = ops.lib.pih_no_alloc_scratch_address()
    assert address, "the array's address is known after the first call"
    return torch.as_tensor(_Array(address, SCRATCH_BYTES // 4), device=DEV)


def test_no_alloc_entry_point_merges_through_the_library_array_call_after_call():
    from pih_b200.kernels import get_ops
    ops = get_ops(torch.device(DEV))
    message = ctypes.create_string_buffer(256)
    g = torch.Generator().manual_seed(5)
    many = [2048] + torch.randint(100, 2048, (30,), generator=g).tolist()        # 31 requests x 32 splits: 7.9 MiB
    calls = [
        # (lengths, keys per split, cluster merge allowed)
        ([2048, 77, 1000, 513, 1999, 640], 64, True),       # up to 32 splits a request: beyond a cluster, so tickets
        ([300, 1999, 64, 1024], 256, False),                # 8 splits, the cluster merge switched off
        (many, 64, True),
        ([2048, 1500], 128, True),
    ]
    for i, (lens, split, cluster) in enumerate(calls):
        p = _problem(41 + i, lens)
        need = _scratch_need(ops, p, split)
        assert need <= SCRATCH_BYTES and (i != 2 or need > 0.93 * SCRATCH_BYTES)
        before = ops.set_attention_cluster_merge(cluster)
        try:
            rc, got = _call_no_alloc(ops, p, split, message)
        finally:
            ops.set_attention_cluster_merge(before)
        assert rc == 0, (rc, message.value)
        torch.cuda.synchronize()
        ops.check_errors()
        torch.testing.assert_close(got.cpu().double(), p["want"], **TOL, msg=lambda m: f"call {i}: {m}")
        scratch = _library_scratch(ops)
        tickets = -(-len(lens) * p["kv_heads"] // 64) * 64
        assert int(scratch[:tickets].abs().max()) == 0              # the kernel leaves its tickets at rest
        assert int(scratch[tickets:need // 4].abs().max()) != 0     # and its partials went through this very array
        # what the next call finds: tickets that are not zero, and NaN wherever a partial result may lie
        scratch.fill_(0x7FC00000)
        torch.cuda.synchronize()


def test_no_alloc_entry_point_refuses_what_does_not_fit():
    from pih_b200.kernels import get_ops
    ops = get_ops(torch.device(DEV))
    message = ctypes.create_string_buffer(256)
    p = _problem(43, [100, 200])
    # a context of a million keys in splits of 64 would need hundreds of MB of partials: beyond the 8 MiB array
    rc, out = _call_no_alloc(ops, p, 64, message, claimed_ctx=1_000_000)
    assert rc == -3 and b"bytes of scratch" in message.value, (rc, message.value)
    # one request more than fits (32 x 32 splits): refused too, by a few per cent
    big = _problem(44, [2048] + [64] * 31)
    rc, out32 = _call_no_alloc(ops, big, 64, message)
    assert rc == -3 and b"bytes of scratch" in message.value, (rc, message.value)
    torch.cuda.synchronize()
    assert float(out.float().abs().max()) == 0.0 and float(out32.float().abs().max()) == 0.0    # nothing was launched
