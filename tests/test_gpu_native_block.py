"""The block issued by one native call gives what the parts give when they issue its kernels one by one."""
import pytest
import torch

import traces

pytestmark = pytest.mark.gpu
PAGE = {"A": 16, "B": 8, "C": 16, "D": 32}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C", "D"])
def test_native_block_equals_the_parts(model_dirs, tiny_configs, name, dtype):
    from pih_b200.engine.factory import create_runner
    requests = traces.make_requests(tiny_configs[name]["vocab_size"], [70, 45, 90, 33, 130], seed=12)
    steps = traces.mixed(requests, seed=3, max_live=3) + traces.tail_decode(requests, tail=6)
    out = {}
    for native in (True, False):
        _, model, cache, runner = create_runner(model_dirs[name], dtype, page_size=PAGE[name],
                                                max_cache_tokens=traces.peak_tokens(steps) + 64, max_requests=4)
        ops = model.rt.ops
        before = ops.native_blocks
        ops.native_blocks = native
        try:
            out[native] = traces.replay(runner, steps)
            ops.check_errors()
        finally:
            ops.native_blocks = before
        assert all(block._native_ok for block in model.blocks)          # the built-in parts are taken
        cache.check()
    for rid in requests:
        a, b = out[True][rid], out[False][rid]
        if dtype == "float32":
            assert torch.equal(a, b), rid                    # the same kernels with the same arguments
        else:
            # steps of more than 16 rows call the library product from two places, which may pick two algorithms
            assert float((a - b).abs().max()) <= 0.03 * float(b.std()), rid


def test_native_block_is_not_taken_for_other_parts(model_dirs, tiny_configs):
    """A block whose parts are not all the built-in ones runs through the parts (checked with a norm subclass)."""
    from pih_b200.engine.factory import create_runner
    from pih_b200.parts.norm import RMSNorm
    _, model, cache, runner = create_runner(model_dirs["A"], "bfloat16", page_size=16, max_cache_tokens=256, max_requests=2)

    class OtherNorm(RMSNorm):
        pass
    block = model.blocks[0]
    block.norm_in.__class__ = OtherNorm
    requests = traces.make_requests(256, [40], seed=2)
    traces.replay(runner, traces.whole(requests))
    assert block._native_ok is False and model.blocks[1]._native_ok is True
    model.rt.ops.check_errors()
