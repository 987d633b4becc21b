"""One key that outweighs all others, placed where a kernel could lose it.

Among hundreds of random keys a dropped key, a dropped tile or a key taken from the wrong page moves the
output by less than the tolerance.  Here one key's score stands 40 above the rest, so the output of the
rows that see it is that key's value and the output of the rows that do not is something else.  The key is
put in the first tile, on both sides of the boundaries between 64-key tiles, pages and splits, in the tile
that holds the step's own new tokens, and just inside and just outside the window of the first and the last
row of a portion; pages that lie wholly before the window read -1 in the block table, as the cache manager
leaves them.  Every family of attention kernels that serving uses at head sizes 64 and 128 runs it: the
TMA-fed split kernel with the cluster merge, with the ticket merge, with the q/k work fused into it, the
cp.async split kernel, the tcgen05 prompt kernel and the mma.sync tile kernel.  The reference is the plain
implementation's attention in float64."""
import math

import pytest
import torch

import plain_impl
from test_gpu_kernels import MMA_TOL, _paged_setup, _step_of

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
HEADS, KV_HEADS, PAGE = 4, 2, 16


@pytest.fixture(scope="module")
def ops():
    from pih_b200.kernels import get_ops
    return get_ops(torch.device(DEV))


# (head_dim, lengths, new rows per request, window, positions of the heavy key)
def _cases():
    out = []
    for D in (64, 128):
        L = 700
        out += [
            (D, [L], [1], None, [0, 3, 63, 64, 255, 256, 639, 640, L - 2, L - 1]),
            (D, [L], [1], 64, [L - 65, L - 64, L - 1]),
            (D, [L], [1], 1, [L - 2, L - 1]),
            (D, [L], [4], None, [63, 64, L - 5, L - 4, L - 1]),          # a decode-like request of four rows
            (D, [L], [4], 100, [L - 104, L - 103, L - 100, L - 4]),
            (D, [2048] * 8, [1] * 8, None, [0, 511, 512, 1023, 1024, 1535, 1536, 2047]),   # batch 8: four splits
            (D, [2048], [1], None, [255, 256, 1791, 1792, 2047]),                     # batch 1: a cluster of eight
            (D, [2048, 5, 300], [1, 1, 1], 512, [1535, 1536, 2047]),
            # a prompt portion deep in the context: rows 1200..1499
            (D, [1500], [300], None, [5, 1199, 1200, 1215, 1216, 1263, 1264, 1498, 1499]),
            (D, [1500], [300], 257, [1200 - 257, 1200 - 256, 1499 - 257, 1499 - 256, 1200, 1499]),
            (D, [900, 130], [70, 130], 40, [829, 830, 831, 860, 899]),
        ]
    return out


CASES = _cases()


def _plant(s, r, far, u, dtype=torch.bfloat16):
    """Key ``far`` of request r, kv head 0, becomes 40 u; returns what was there."""
    page = int(s["table_full"][r, far // PAGE])
    old = s["ks"][r][far, 0].clone()
    s["ks"][r][far, 0] = (u * 40.0).to(dtype)
    s["cache"][page, 0, 0, far % PAGE] = s["ks"][r][far, 0].to(DEV)
    return page, old


def _unplant(s, r, far, page, old):
    s["ks"][r][far, 0] = old
    s["cache"][page, 0, 0, far % PAGE] = old.to(DEV)


def _run(ops, kind, s, D, lens, new, window, scale):
    step = _step_of(lens, new)
    kw = dict(heads=HEADS, kv_heads=KV_HEADS, head_dim=D, kv_cache=s["cache"], block_table=s["table"], step=step,
              scale=scale, window=window or 0)
    if kind == "fused":
        # raw rows [q | k | v] of the step's tokens; no norm, no rotation: the kernel appends k and v itself
        rows = sum(new)
        k_new = torch.cat([s["ks"][r][lens[r] - new[r]:] for r in range(len(lens))]).reshape(rows, -1)
        v_new = torch.cat([s["vs"][r][lens[r] - new[r]:] for r in range(len(lens))]).reshape(rows, -1)
        qkv = torch.cat([s["q"], k_new.to(DEV), v_new.to(DEV)], dim=1).contiguous()
        slots = []
        for r in range(len(lens)):
            for j in range(lens[r] - new[r], lens[r]):
                slots.append((int(s["table_full"][r, j // PAGE]), j % PAGE))
        for pg, off in slots:                                # the step's own keys are not in the cache yet
            s["cache"][pg, :, :, off] = 0
        out = ops.qk_attention_fused(qkv, q_norm=None, k_norm=None, eps=0.0, rope_table=None, rotary_dim=0,
                                     write_kv=True, **kw)
        assert out is not None, "the fused decode attention refused a shape that serving gives it"
        return out
    return ops.paged_attention_mma(s["q"], **kw)


@pytest.mark.parametrize("case", CASES, ids=[f"d{c[0]}-r{len(c[1])}-n{max(c[2])}-w{c[3]}" for c in CASES])
def test_one_heavy_key_is_found_or_masked_exactly(ops, case):
    D, lens, new, window, fars = case
    s = _paged_setup(torch.bfloat16, lens, new, HEADS, KV_HEADS, D, PAGE, seed=17)
    s["table_full"] = s["table"].clone()
    g = torch.Generator().manual_seed(3)
    u = torch.randn(D, generator=g)
    u = u / u.norm()
    # every row's query head 0 points along u with the length of a random query
    q = s["q"].reshape(sum(new), HEADS, D)
    q[:, 0] = (u * math.sqrt(D)).to(torch.bfloat16).to(DEV)
    row = 0
    for r in range(len(lens)):
        s["qs"][r][:, 0] = (u * math.sqrt(D)).to(torch.bfloat16)
        row += new[r]
    if window is not None:                                   # pages wholly before every row's window were given back
        for r in range(len(lens)):
            first = max(0, lens[r] - new[r] - window + 1) // PAGE
            s["table"][r, :first] = -1
    scale = 1.0 / math.sqrt(D)
    decode_like = all(n * (HEADS // KV_HEADS) <= 16 for n in new)
    kinds = ["cluster", "fetched", "tickets", "fused", "cp.async"] if decode_like else ["tcgen05", "mma.sync"]
    for far in fars:
        planted = [(r,) + _plant(s, r, far, u) for r in range(len(lens)) if 0 <= far < lens[r]]
        try:
            ref = torch.cat([plain_impl.attention_rows(s["qs"][r], range(lens[r] - new[r], lens[r]), s["ks"][r],
                                                        s["vs"][r], scale, window).reshape(new[r], -1)
                             for r in range(len(lens))])
            for kind in kinds:
                modern = kind not in ("cp.async", "mma.sync")
                ops.tcgen05_attention = ops.tma_attention = modern
                ops.set_attention_cluster_merge("fetched" if kind == "fetched" else kind != "tickets")
                try:
                    out = _run(ops, kind, s, D, lens, new, window, scale)
                finally:
                    ops.tcgen05_attention = ops.tma_attention = True
                    ops.set_attention_cluster_merge(True)
                ops.check_errors()
                torch.testing.assert_close(out.cpu().double(), ref, **MMA_TOL, msg=lambda m: f"{kind}, key {far}: {m}")
                row = 0
                for r in range(len(lens)):
                    for i in range(new[r]):
                        p = lens[r] - new[r] + i
                        sees = far < lens[r] and far <= p and (window is None or far > p - window)
                        if far < lens[r]:
                            near = float((out[row + i, :D].cpu().double() - s["vs"][r][far, 0].double()).abs().max())
                            assert (near < 0.06) == sees, (kind, far, r, p, near)
                    row += new[r]
        finally:
            for r, page, old in planted:
                _unplant(s, r, far, page, old)
