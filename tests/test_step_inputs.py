"""The step packer on the CPU: what one mixed step's device inputs hold.

Every field is checked against a restatement in plain Python of what a step needs: positions
and cache slots of each token, the row tiles of prompt portions, the single decoded tokens,
the rows whose logits are wanted, padding requests that write nothing, and the host-side
figures that launches are sized from.
"""
import random

import pytest
import torch

from einf_b200 import ops
from einf_b200.engine.batch import Q_TILE, BatchError, StepInputBuilder


class _Request:
    def __init__(self, tokens, start, table, need_sample=True, state_slot=-1):
        self.input_token_ids = tokens
        self.start_position = start
        self.block_tables = [table]
        self.need_sample = need_sample
        self.state_slot = state_slot


def _builder(page=8, pages=64, width=40, max_tokens=512, max_requests=8, window=None, vocab=1000):
    return StepInputBuilder(torch.device("cpu"), page, [pages], [window], vocab, width, max_tokens, max_requests)


def _tables(rng, lengths, page, pages):
    free = list(range(pages))
    rng.shuffle(free)
    return [[free.pop() for _ in range(-(-n // page))] for n in lengths]


@pytest.mark.parametrize("seed", range(6))
def test_a_mixed_step_is_laid_out_as_the_kernels_read_it(seed):
    rng = random.Random(seed)
    page = rng.choice([4, 8, 16])
    builder = _builder(page=page, pages=256, width=64)
    shapes = [(0, 150), (37, 1), (129, 2), (200, 1), (5, 130)][: rng.randint(2, 5)]
    rng.shuffle(shapes)
    tables = _tables(rng, [s + n for s, n in shapes], page, 256)
    requests = [
        _Request([rng.randrange(1000) for _ in range(n)], s, t, need_sample=rng.random() < 0.7, state_slot=i + 3)
        for i, ((s, n), t) in enumerate(zip(shapes, tables))
    ]
    pad_to = len(requests) + rng.choice([0, 0, 2])
    ctx, rows = builder.build(requests, pad_requests_to=pad_to)

    tokens, positions, seq, slots, singles, tiles, wanted = [], [], [], [], [], [], []
    cursor = 0
    for i, r in enumerate(requests):
        n = len(r.input_token_ids)
        if n == 1:
            singles.append(cursor)
        else:
            for first in range(0, n, Q_TILE):
                tiles.append([i, cursor + first, min(Q_TILE, n - first), r.start_position + first])
        for t, token in enumerate(r.input_token_ids):
            pos = r.start_position + t
            tokens.append(token)
            positions.append(pos)
            seq.append(i)
            slots.append(r.block_tables[0][pos // page] * page + pos % page)
        if r.need_sample:
            wanted.append(cursor + n - 1)
        cursor += n
    for extra in range(pad_to - len(requests)):
        tokens.append(0)
        positions.append(0)
        seq.append(len(requests) + extra)
        slots.append(-1)
        singles.append(cursor)
        wanted.append(cursor)
        cursor += 1

    assert ctx.num_tokens == cursor and ctx.num_requests == max(pad_to, len(requests))
    assert ctx.token_ids.tolist() == tokens
    assert ctx.positions.tolist() == positions
    assert ctx.seq_of_token.tolist() == seq
    assert ctx.slots[0].tolist() == slots
    assert ctx.single_tokens.tolist() == singles
    assert ctx.q_tiles.tolist() == tiles
    assert ctx.logit_rows.tolist() == wanted
    assert ctx.q_start.tolist()[: len(requests) + 1] == [0] + [
        sum(len(r.input_token_ids) for r in requests[: i + 1]) for i in range(len(requests))
    ]
    assert ctx.context_lens.tolist()[: len(requests)] == [r.start_position + len(r.input_token_ids) for r in requests]
    assert ctx.state_slots.tolist() == [r.state_slot for r in requests] + [-1] * (pad_to - len(requests))
    for i, r in enumerate(requests):
        row = ctx.block_tables[0][i].tolist()
        assert row[: len(r.block_tables[0])] == r.block_tables[0]
        assert all(p == -1 for p in row[len(r.block_tables[0]):])
    # the rows of each request's logits, in the order of the requests
    at = 0
    for r, (first, count) in zip(requests, rows):
        assert (first, count) == (at, 1 if r.need_sample else 0)
        at += count
    # host copies that size launches
    assert ctx.q_lens[: len(requests)] == tuple(len(r.input_token_ids) for r in requests)
    assert ctx.start_positions[: len(requests)] == tuple(r.start_position for r in requests)
    assert ctx.max_q_len == max(len(r.input_token_ids) for r in requests)
    assert ctx.max_context_len == max(r.start_position + len(r.input_token_ids) for r in requests)
    portions = [r.start_position for r in requests if len(r.input_token_ids) > 1]
    assert ctx.max_portion_start == max(portions, default=0)
    assert ctx.decode_only == (not portions)
    assert int(ctx.status) == 0


def test_wanted_places_come_in_the_order_given():
    builder = _builder()
    a = _Request([1, 2, 3, 4, 5], 0, [3])
    b = _Request([9], 11, [7, 1], need_sample=False)
    ctx, rows = builder.build([a, b], want=[[4, 0, 2], []])
    assert ctx.logit_rows.tolist() == [4, 0, 2]
    assert rows == [(0, 3), (3, 0)]
    ctx, rows = builder.build([a, b], want=[[], [0]])
    assert ctx.logit_rows.tolist() == [5]
    assert rows == [(0, 0), (0, 1)]


def test_a_windowed_group_may_miss_the_pages_behind_its_window():
    builder = _builder(page=8, window=16)
    # positions 40..41: keys from 40 - 16 + 1 = 25 on, so pages 0 to 2 may be gone
    request = _Request([5, 6], 40, [-1, -1, -1, 9, 4, 2])
    ctx, _ = builder.build([request])
    assert ctx.block_tables[0][0].tolist()[:6] == [-1, -1, -1, 9, 4, 2]
    assert ctx.slots[0].tolist() == [2 * 8 + 0, 2 * 8 + 1]
    with pytest.raises(BatchError, match="missing from its block table"):
        builder.build([_Request([5, 6], 40, [-1, -1, -1, -1, 4, 2])])


def test_the_prefix_bucket_is_what_a_prefill_launch_keeps_of_the_contexts():
    assert [ops.prefill_prefix_bucket(n) for n in (None, 0, 511, 512, 1023, 1024, 10 ** 6)] == [1, 1, 1, 4, 4, 8, 8]


def test_the_context_bucket_is_what_a_decode_launch_keeps_of_the_contexts():
    assert [ops.decode_context_bucket(n) for n in (None, 0, 1, 4096, 4097, 8192, 8193, 32768, 100000)] == [
        4096, 4096, 4096, 4096, 8192, 8192, 16384, 32768, 131072]


def test_the_decode_attention_cuts_the_keys_by_an_estimate_of_each_shape():
    """``decode_plan``'s choice with figures like a B200's given by hand (clusters of a size that
    the device holds at once at head size 64 and 128; 148 SMs): a few requests get clusters of 16,
    from tens of thousands of tokens on several of them per token; eight requests of 4,096 tokens
    keep clusters of eight (sixteen clusters of 16 do not fit) and at 32,768 tokens get four
    clusters of four; many requests get small clusters and never more than one a token."""
    held = {64: {16: 14, 8: 30, 7: 36, 6: 44, 5: 54, 4: 66, 3: 96, 2: 148, 1: 296},
            128: {16: 7, 8: 15, 7: 18, 6: 22, 5: 27, 4: 33, 3: 48, 2: 74, 1: 148}}

    def plan(tokens, heads, kv_heads, size, context):
        return ops._plan_decode(tokens, heads, kv_heads, size, 16, ops.decode_context_bucket(context),
                                room=lambda head_size, cluster: held[head_size][cluster], sms=148)[1:]

    assert plan(1, 14, 2, 64, 4096) == (16, 1)
    assert plan(4, 14, 2, 64, 4096) == (16, 1)
    assert plan(7, 14, 2, 64, 4096) == (8, 1)          # clusters of 16 would share SMs
    assert plan(8, 14, 2, 64, 4096) == (8, 1)
    assert plan(8, 14, 2, 64, 8192) == (8, 1)
    assert plan(8, 14, 2, 64, 32768) == (4, 4)
    assert plan(1, 14, 2, 64, 32768) == (16, 4)
    assert plan(64, 14, 2, 64, 4096) == (2, 1)
    assert plan(1, 28, 4, 128, 4096) == (16, 1)
    assert plan(8, 28, 4, 128, 32768) == (4, 1)        # 32 pairs of one-CTA-per-SM blocks: nothing larger fits
    assert plan(64, 28, 4, 128, 4096) == (1, 1)
    for tokens in (1, 2, 3, 8, 16, 64, 300):
        for size, heads, kv_heads in ((64, 14, 2), (128, 12, 2), (128, 28, 4)):
            for context in (100, 4096, 20000, 131072):
                cluster, splits = plan(tokens, heads, kv_heads, size, context)
                pairs = tokens * kv_heads
                assert cluster == 1 and splits == 1 or pairs * splits <= held[size][cluster]
