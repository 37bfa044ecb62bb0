"""Streaming base helpers (vectors: axlearn/audio/streaming/streaming_base_test.py:57-111)."""

import pytest

from axlearn_b200.audio.streaming import convolutions as sc
from axlearn_b200.audio.streaming.streaming_base import (
    StreamingBase,
    compute_decoder_segment_pad,
    compute_encoder_segment_pad,
    config_method,
    next_segment_pos,
)
from axlearn_b200.common.config import config_class
from axlearn_b200.common.module import Module


class MockLayer(StreamingBase, Module):
    @config_class
    class Config(Module.Config):
        in_stride: int = 1
        out_stride: int = 1
        segment_pad: int = 0

    @config_method
    def in_stride(cls, cfg):  # pylint: disable=no-self-argument
        return cfg.in_stride

    @config_method
    def out_stride(cls, cfg):  # pylint: disable=no-self-argument
        return cfg.out_stride

    @config_method
    def segment_pad(cls, cfg):  # pylint: disable=no-self-argument
        return cfg.segment_pad


def _cfg(**kw):
    return MockLayer.default_config().set(name="m", **kw)


@pytest.mark.parametrize("layers,expected", [
    ([], 0),
    ([_cfg(segment_pad=5, in_stride=2)], 5),
    ([_cfg(segment_pad=2, in_stride=4), _cfg(segment_pad=3, in_stride=1)], 12),
    ([_cfg(segment_pad=1, in_stride=2), _cfg(segment_pad=1, in_stride=3), _cfg(segment_pad=160, in_stride=160)], 960),
])
def test_encoder_segment_pad(layers, expected):
    assert compute_encoder_segment_pad(layers) == expected
    assert compute_encoder_segment_pad([c.instantiate(parent=None) for c in layers]) == expected


@pytest.mark.parametrize("layers,expected", [
    ([], 0),
    ([_cfg(segment_pad=5, out_stride=2)], 5),
    ([_cfg(segment_pad=2, out_stride=4), _cfg(segment_pad=10, out_stride=1)], 3),
    ([_cfg(segment_pad=2, out_stride=160), _cfg(segment_pad=1, out_stride=3), _cfg(segment_pad=2, out_stride=2)], 2),
])
def test_decoder_segment_pad(layers, expected):
    assert compute_decoder_segment_pad(layers) == expected


@pytest.mark.parametrize("current_len,segment_pad,stride,expected", [
    (0, 0, 1, (0, 0)), (5, 3, 1, (8, 3)), (5, 0, 4, (8, 3)), (5, 3, 4, (8, 3)), (10, 5, 8, (16, 6)),
    (960, 960, 960, (1920, 960)),
])
def test_next_segment_pos(current_len, segment_pad, stride, expected):
    assert next_segment_pos(current_len, segment_pad=segment_pad, stride=stride) == expected


def test_convolutions_answer_from_config_and_instance():
    cfg = sc.CausalConv1D.default_config().set(name="c", window=3, strides=2, input_dim=4, output_dim=4)
    assert sc.CausalConv1D.in_stride(cfg) == 2 and sc.CausalConv1D.out_stride(cfg) == 1
    layer = cfg.instantiate(parent=None)
    assert layer.in_stride() == 2 and layer.segment_pad() == sc.CausalConv1D.segment_pad(cfg) == layer.cache_size()
    up = sc.CausalConv1DTranspose.default_config().set(name="u", window=4, strides=2, input_dim=4, output_dim=4)
    # w=4, s=2: padding (3, 1) in output frames -> one input frame between segments.
    assert sc.CausalConv1DTranspose.segment_pad(up) == 1 and sc.CausalConv1DTranspose.out_stride(up) == 2
    assert compute_encoder_segment_pad([cfg, cfg]) == max(layer.segment_pad(), layer.segment_pad() * 2)
    assert compute_decoder_segment_pad([up, up]) == 1
