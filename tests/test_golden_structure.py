"""Parameter names and shapes of the flagship configs against the reference's golden init listings
(axlearn/experiments/testdata/axlearn.experiments.text.gpt.c4_trainer/*_init.txt).  The listings
give per-layer shapes: the leading layer dim of repeated stacks and the leading 3 of the fused QKV
projection are not part of them."""

import pytest

from axlearn_b200.common.utils import flatten_items
from axlearn_b200.experiments.text.gpt import envy, fuji

FUJI_7B_V2 = """
decoder/emb/token_emb/weight 32768,4096
decoder/transformer/repeat/layer/self_attention/norm/scale
decoder/transformer/repeat/layer/self_attention/attention/i_proj/i_proj/qkv_proj/weight 4096,32,128
decoder/transformer/repeat/layer/self_attention/attention/o_proj/weight 4096,32,128
decoder/transformer/repeat/layer/feed_forward/norm/scale
decoder/transformer/repeat/layer/feed_forward/linear1_0/weight 4096,11008
decoder/transformer/repeat/layer/feed_forward/linear1_1/weight 4096,11008
decoder/transformer/repeat/layer/feed_forward/linear2/weight 11008,4096
decoder/output_norm/scale
"""

FUJI_70B_V2 = """
decoder/emb/token_emb/weight 32768,8192
decoder/transformer/repeat/layer/self_attention/norm/scale
decoder/transformer/repeat/layer/self_attention/attention/i_proj/i_proj/qkv_proj/weight 8192,80,128
decoder/transformer/repeat/layer/self_attention/attention/o_proj/weight 8192,64,128
decoder/transformer/repeat/layer/feed_forward/norm/scale
decoder/transformer/repeat/layer/feed_forward/linear1_0/weight 8192,28672
decoder/transformer/repeat/layer/feed_forward/linear1_1/weight 8192,28672
decoder/transformer/repeat/layer/feed_forward/linear2/weight 28672,8192
decoder/output_norm/scale
decoder/lm_head/weight 32768,8192
"""

ENVY_SWITCH_BASE = """
decoder/emb/token_emb/weight 32768,1536
decoder/transformer/repeat/layer/layer0/self_attention/norm/scale
decoder/transformer/repeat/layer/layer0/self_attention/attention/i_proj/i_proj/qkv_proj/weight 1536,36,128
decoder/transformer/repeat/layer/layer0/self_attention/attention/o_proj/weight 1536,12,128
decoder/transformer/repeat/layer/layer0/self_attention/attention/scale_query/norm/scale
decoder/transformer/repeat/layer/layer0/self_attention/attention/scale_key/norm/scale
decoder/transformer/repeat/layer/layer0/feed_forward/prenorm/scale
decoder/transformer/repeat/layer/layer0/feed_forward/postnorm/scale
decoder/transformer/repeat/layer/layer0/feed_forward/linear1_0/weight 1536,6144
decoder/transformer/repeat/layer/layer0/feed_forward/linear1_1/weight 1536,6144
decoder/transformer/repeat/layer/layer0/feed_forward/linear2/weight 6144,1536
decoder/transformer/repeat/layer/layer1/self_attention/norm/scale
decoder/transformer/repeat/layer/layer1/self_attention/attention/i_proj/i_proj/qkv_proj/weight 1536,36,128
decoder/transformer/repeat/layer/layer1/self_attention/attention/o_proj/weight 1536,12,128
decoder/transformer/repeat/layer/layer1/self_attention/attention/scale_query/norm/scale
decoder/transformer/repeat/layer/layer1/self_attention/attention/scale_key/norm/scale
decoder/transformer/repeat/layer/layer1/feed_forward/gate_weight 1536,128
decoder/transformer/repeat/layer/layer1/feed_forward/wo_weight 128,6144,1536
decoder/transformer/repeat/layer/layer1/feed_forward/wi_0_weight 128,1536,6144
decoder/transformer/repeat/layer/layer1/feed_forward/wi_1_weight 128,1536,6144
decoder/transformer/repeat/layer/layer1/feed_forward/prenorm/scale
decoder/transformer/repeat/layer/layer1/feed_forward/postnorm/scale
decoder/output_norm/scale
"""


def _golden(text):
    out = {}
    for line in text.strip().splitlines():
        name, _, shape = line.partition(" ")
        out[name] = tuple(int(v) for v in shape.split(",")) if shape else None
    return out


def _ours(model_cfg, num_layers):
    model = model_cfg.clone(name="model").instantiate(parent=None)
    specs = flatten_items(model.create_parameter_specs_recursively(), is_leaf=lambda x: hasattr(x, "mesh_axes"))
    out = {}
    for path, spec in specs:
        shape = tuple(spec.shape)
        if "/repeat/" in path:
            assert shape[0] == num_layers, (path, shape)
            shape = shape[1:]
        if path.endswith("qkv_proj/weight") and len(shape) == 4:        # fused multi-head: [3, D, N, H]
            assert shape[0] == 3
            shape = shape[1:]
        out[path] = shape
    return out


@pytest.mark.parametrize("config_name,golden,layers", [("fuji-7B-v2-flash", FUJI_7B_V2, 32), ("fuji-70B-v2-flash", FUJI_70B_V2, 80)])
def test_fuji_matches_reference_listing(config_name, golden, layers):
    cfg = fuji.trainer_configs()[config_name]()
    ours, want = _ours(cfg.model, layers), _golden(golden)
    assert list(ours) == list(want) or set(ours) == set(want)
    for name, shape in want.items():
        if shape is not None:
            assert ours[name] == shape, name
        else:
            assert len(ours[name]) == 1, name


def test_envy_switch_base_matches_reference_listing():
    ours, want = _ours(envy.preset("Switch-Base"), 6), _golden(ENVY_SWITCH_BASE)      # 12 layers = 6 x (dense, sparse)
    assert set(ours) == set(want), sorted(set(ours) ^ set(want))
    for name, shape in want.items():
        if shape is not None:
            assert ours[name] == shape, name


def test_fuji_initializers_match_reference_listing():
    """The listing also names the initialiser of every weight: ``normal(0, 1 / fan_out)`` for the
    token embedding, ``normal(0, 1 / fan_in)`` elsewhere, with fan axes in per-layer coordinates
    ``qkv_proj: in 0, out (1, 2)``, ``o_proj: in (1, 2), out 0`` and ``in -2, out -1`` for the rest."""
    cfg = fuji.trainer_configs()["fuji-7B-v2-flash"]()
    model = cfg.model.clone(name="model").instantiate(parent=None)
    specs = dict(flatten_items(model.create_parameter_specs_recursively(), is_leaf=lambda x: hasattr(x, "mesh_axes")))

    def fan(path):
        spec = specs[path]
        batch = len(spec.fan_axes.batch_axis)
        rank = len(spec.shape)
        norm = lambda a: tuple(sorted((i % rank) - batch for i in ((a,) if isinstance(a, int) else a)))
        return norm(spec.fan_axes.in_axis), norm(spec.fan_axes.out_axis)

    layer = "decoder/transformer/repeat/layer/"
    assert fan(layer + "self_attention/attention/i_proj/i_proj/qkv_proj/weight") == ((0,), (1, 2))
    assert fan(layer + "self_attention/attention/o_proj/weight") == ((1, 2), (0,))
    assert fan(layer + "feed_forward/linear2/weight") == ((0,), (1,))
    assert fan("decoder/emb/token_emb/weight") == ((0,), (1,))

    def weight_init(path):
        init = specs[path].initializer
        init_cfg = init.config if hasattr(init, "config") else init
        rule = init_cfg.init_by_param_name[".*weight$"]
        return rule.fan, rule.distribution, rule.scale

    assert weight_init("decoder/emb/token_emb/weight") == ("fan_out", "normal", 1.0)
    assert weight_init(layer + "feed_forward/linear1_0/weight") == ("fan_in", "normal", 1.0)
    assert weight_init(layer + "self_attention/attention/o_proj/weight") == ("fan_in", "normal", 1.0)
