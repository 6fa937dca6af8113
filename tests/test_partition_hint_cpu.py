"""The host-side test that decides whether a decode launch may keep (sequence, KV head) units whole
(PACE_ATTN_WHOLE_UNITS): the arithmetic the kernel applies on the device, applied to the host mirror."""
from pace_b200.ops.backends.b200 import even_lengths


def test_benchmark_batch_keeps_units_whole():
    # batch 32 x 8 KV heads on 2 x 148 thread blocks: one unit each, 1.24x an even share
    assert even_lengths([519 + i for i in range(32)], 8, 128, 64, None, sms=148)
    assert even_lengths([576] * 32, 8, 128, 64, None, sms=148)


def test_small_or_ragged_batches_are_cut():
    assert not even_lengths([128, 1024, 577, 300], 8, 128, 64, None, sms=148)     # 32 units on 296 blocks
    assert not even_lengths([64] * 31 + [8192], 8, 128, 64, None, sms=148)        # one long sequence
    assert not even_lengths([], 8, 128, 64, None, sms=148)


def test_two_units_per_block():
    # 64 sequences: 512 units, two per block on 256 of 296 blocks -> 2 x 9 x 296 against 512 x 9 x 1.3
    assert even_lengths([570] * 64, 8, 128, 64, None, sms=148)
    # 40 sequences: 320 units, two per block on 160 blocks only -> too uneven
    assert not even_lengths([570] * 40, 8, 128, 64, None, sms=148)


def test_small_pages_count_chunks_of_several_pages():
    # 16-token pages: four pages per 64-key chunk
    assert even_lengths([520] * 32, 8, 128, 16, None, sms=148)
