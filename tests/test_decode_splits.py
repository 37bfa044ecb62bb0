"""KV-split heuristic of paged decode attention (pure arithmetic; runs without a GPU)."""

import math

import pytest

from axlearn_b200.ops import decode_ops


@pytest.mark.parametrize("batch,kv,group,tokens,want", [
    (32, 32, 1, 2048, 1),      # 1024 CTAs fit the 1184 resident ones: one wave, no split
    (64, 32, 1, 2048, 4),      # 2048 CTAs = 1.73 waves; 4 splits = 6.92 waves of 7
    (16, 4, 1, 2048, 10),      # small grid: split until about four CTAs per SM
    (64, 8, 4, 2048, 9),       # row kernel (two resident CTAs per SM): 9 splits = 3.89 waves of 4
    (16, 8, 4, 2048, 9),
    (64, 16, 2, 2048, 4),      # two query heads per KV head run one per CTA
    (1, 32, 1, 64, 1),         # never below 8 pages per split
])
def test_default_splits(batch, kv, group, tokens, want, monkeypatch):
    monkeypatch.delenv("AXB_DECODE_ATTN", raising=False)
    assert decode_ops.default_splits(batch, kv, group, tokens, 16) == want


def test_last_wave_is_nearly_full_once_past_one_wave(monkeypatch):
    monkeypatch.delenv("AXB_DECODE_ATTN", raising=False)
    for batch in (24, 40, 48, 64, 96, 128, 200):
        for kv, group in ((32, 1), (8, 4), (16, 2)):
            s = decode_ops.default_splits(batch, kv, group, 4096, 16)
            ctas, resident = decode_ops._kernel_shape(batch, kv, group)  # pylint: disable=protected-access
            x = ctas * s / (148 * resident)
            assert 1 <= s <= 32
            if x > 1:
                assert x / math.ceil(x) >= 0.85, (batch, kv, group, s, x)


def test_kernel_shape_follows_the_environment(monkeypatch):
    monkeypatch.delenv("AXB_DECODE_ATTN", raising=False)
    assert decode_ops._kernel_shape(64, 8, 4) == (128, 2)        # pylint: disable=protected-access
    assert decode_ops._kernel_shape(4, 8, 4) == (128, 8)         # few row CTAs: one query head per CTA
    assert decode_ops._kernel_shape(8, 2, 4) == (16, 2)          # KV heads not a multiple of 4: 4 heads per CTA
    monkeypatch.setenv("AXB_DECODE_ATTN", "head")
    assert decode_ops._kernel_shape(64, 8, 4) == (512, 2)        # pylint: disable=protected-access
    monkeypatch.setenv("AXB_DECODE_ATTN", "head1")
    assert decode_ops._kernel_shape(64, 8, 4) == (2048, 8)       # pylint: disable=protected-access
