"""The packed batch of a step on the host: what padding to a larger shape puts where, and the runner's choice of
shapes.  (What the kernels make of padding is tested on the GPU.)"""
import pytest
import torch

from pih_b200.cache import CacheManager
from pih_b200.engine.batch import PAD_SLOT, BatchBuilder, StepEntry
from pih_b200.engine.runner import ModelRunner, _requests_bucket, _rows_bucket
from pih_b200.parts import PagedKVNeed


def _cache(page_size=4, num_pages=32, max_requests=4):
    needs = [PagedKVNeed(2, 8, None), PagedKVNeed(2, 8, 6)]                 # two cache groups: all keys, a window
    return CacheManager(needs, [None, None], page_size=page_size, num_pages=num_pages, max_requests=max_requests,
                        device=torch.device("cpu"), dtype=torch.float32)


def test_padding_is_marked_in_the_data_and_changes_nothing_of_the_real_step():
    cache = _cache()
    entries = [StepEntry("a", [5, 6, 7], [2]), StepEntry("b", [9], [0]), StepEntry("c", [1, 2], [])]
    for e in entries:
        cache.add_request(e.rid)
        cache.append(e.rid, len(e.tokens))
    builder = BatchBuilder(torch.device("cpu"))
    plain = builder.build(entries, cache, width=8)
    keep = {k: getattr(plain, k).clone() for k in ("token_ids", "positions", "request_of_row", "logit_rows", "cu_q",
                                                    "q_start", "ctx_len", "state_slots", "meta")}
    keep_tables = [t.clone() for t in plain.block_tables]
    keep_slots = [t.clone() for t in plain.slot_mappings]
    padded = builder.build(entries, cache, width=8, pad=(16, 4, 4))
    T, R, S = 6, 3, 2
    assert (padded.num_rows, padded.num_requests, padded.num_logit_rows) == (16, 4, 4) and padded.padded
    assert (padded.real_rows, padded.real_requests, padded.real_logit_rows) == (T, R, S) and not plain.padded
    # the real step is there unchanged
    for k, n in (("token_ids", T), ("positions", T), ("request_of_row", T), ("logit_rows", S), ("cu_q", R + 1),
                 ("q_start", R), ("ctx_len", R), ("state_slots", R)):
        assert torch.equal(getattr(padded, k)[:n], keep[k]), k
    assert torch.equal(padded.meta, keep["meta"])                      # (longest context, rows, requests, wanted): the real ones
    for g in range(2):
        assert torch.equal(padded.block_tables[g][:R], keep_tables[g])
        assert torch.equal(padded.slot_mappings[g][:T], keep_slots[g])
    # rows of padding: token 0, position 0, no request, the slot that says "write nothing"
    assert padded.token_ids[T:].tolist() == [0] * 10 and padded.positions[T:].tolist() == [0] * 10
    assert padded.request_of_row[T:].tolist() == [-1] * 10
    assert all(sm[T:].tolist() == [PAD_SLOT] * 10 for sm in padded.slot_mappings)
    # a request of padding: no rows, length 0, no state slot, no pages
    assert padded.cu_q.tolist() == [0, 3, 4, 6, 6] and padded.host_cu_q == [0, 3, 4, 6, 6]
    assert padded.q_start[R:].tolist() == [0] and padded.ctx_len[R:].tolist() == [0] and padded.state_slots[R:].tolist() == [-1]
    assert all(t[R:].eq(-1).all() for t in padded.block_tables)
    # a wanted row of padding repeats row 0
    assert padded.logit_rows.tolist() == [2, 3, 0, 0]
    with pytest.raises(ValueError, match="padded to less"):
        builder.build(entries, cache, width=8, pad=(4, 4, 4))


def test_buckets():
    assert [_rows_bucket(n) for n in (1, 16, 17, 33, 100, 129, 500, 513, 2048, 4097, 9000)] == \
        [16, 16, 32, 64, 128, 192, 512, 768, 2048, 6144, 10240]
    assert [_requests_bucket(n) for n in (1, 2, 3, 4, 5, 17, 32, 33)] == [1, 2, 4, 4, 8, 32, 32, 64]


def test_the_runner_keys_steps_by_their_padded_shape():
    runner = ModelRunner.__new__(ModelRunner)
    runner.cuda_graphs, runner.device, runner.pad_steps = True, torch.device("cuda"), True
    decode = lambda n: [StepEntry(i, [1], [0]) for i in range(n)]
    assert runner._graph_key(decode(5)) == ("decode", 5) and runner._graph_key(decode(16)) == ("decode", 16)
    assert runner._graph_key(decode(17)) == ("decode", 24) and runner._graph_key(decode(33)) == ("decode", 40)
    assert runner._padding(("decode", 24), decode(17)) == (24, 24, 24) and runner._padding(("decode", 5), decode(5)) is None
    mixed = decode(3) + [StepEntry("p", list(range(200)), [199])]
    assert runner._graph_key(mixed) == ("padded", 256, 4, 4, True, True)
    # nobody wants a row: no head product; only portions: no decode attention
    assert runner._graph_key([StepEntry("p", list(range(300)), [])]) == ("padded", 384, 1, 0, False, True)
    # a request that wants a row in the middle (the replay program): run as it is
    assert runner._graph_key([StepEntry("p", list(range(300)), [7])]) is None
    runner.pad_steps = False                                # a model with a part that does not allow padding
    assert runner._graph_key(mixed) == ("step", (1, 1, 1, 200), (1, 1, 1, 1))
    assert runner._graph_key(decode(17)) == ("decode", 17)
