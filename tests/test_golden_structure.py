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


def test_fuji_7b_trainer_hyperparameters_match_reference_config_dump():
    """Scalar settings of ``fuji-7B-v2-flash`` as listed in the reference's golden config dump
    (``fuji-7B-v2-flash.txt``, ``path: value`` lines)."""
    cfg = fuji.trainer_configs()["fuji-7B-v2-flash"]()
    flat = cfg.to_flat_dict(omit_default_values=set())
    want = {
        "max_step": 524288,
        "checkpointer.keep_every_n_steps": 50000,
        "checkpointer.save_policy.n": 5000,
        "learner.optimizer.args[0].max_norm": 1,
        "learner.optimizer.args[1].b1": 0.9,
        "learner.optimizer.args[1].b2": 0.95,
        "learner.optimizer.args[1].eps": 1e-8,
        "learner.optimizer.args[1].learning_rate": 3e-4,
        "learner.optimizer.args[1].weight_decay": 0.1,
        "learner.optimizer.args[1].update_schedule.alpha": 0.1,
        "learner.optimizer.args[1].update_schedule.max_step": 524288,
        "learner.optimizer.args[1].update_schedule.peak_lr": 1.0,
        "learner.optimizer.args[1].update_schedule.warmup_steps": 2000,
        "mesh_axis_names[0]": "pipeline", "mesh_axis_names[3]": "fsdp", "mesh_axis_names[5]": "model",
        "mesh_shape[1]": -1, "mesh_shape[3]": 8,
        "model.decoder.dim": 4096,
        "model.decoder.vocab_size": 32768,
        "model.decoder.transformer.num_layers": 32,
        "model.decoder.output_norm.eps": 1e-5,
        "model.decoder.transformer.layer.feed_forward.norm.eps": 1e-5,
        "model.decoder.transformer.layer.self_attention.norm.eps": 1e-5,
        "model.decoder.transformer.layer.self_attention.attention.num_heads": 32,
        "model.decoder.transformer.layer.self_attention.attention.input_linear.rope_pos_emb_layer.theta": 10000.0,
    }
    missing = [k for k in want if k not in flat]
    assert not missing, missing
    wrong = {k: (flat[k], v) for k, v in want.items() if flat[k] != v}
    assert not wrong, wrong
    import torch

    assert flat["train_dtype"] == torch.bfloat16 and flat["model.dtype"] == torch.float32
    assert flat["input.global_batch_size"] * flat["input.source_length"] == 4 * 2 ** 20      # 4M tokens per batch


@pytest.mark.parametrize("name,want", [
    ("fuji-70B-v2-flash", dict(max_step=524288, lr=1.5e-4, mesh=(1, 1, 1, -1, 1, 1), dim=8192, heads=64, kv=8, layers=80,
                               vocab=32768, theta=1e4, seq=4096, ffn=28672, head=True)),
    ("fuji-7B-v3-flash", dict(max_step=983040, lr=3e-4, mesh=(1, -1, 1, 8, 1, 1), dim=4096, heads=32, kv=8, layers=32,
                              vocab=131072, theta=5e5, seq=8192, ffn=11008, head=False)),
    ("fuji-1B-v3-flash", dict(max_step=983040, lr=3e-4, mesh=(1, -1, 1, 8, 1, 1), dim=2048, heads=32, kv=8, layers=16,
                              vocab=131072, theta=5e5, seq=8192, ffn=8192, head=False)),
    ("fuji-70B-v3-flash", dict(max_step=983040, lr=1.5e-4, mesh=(1, 1, 1, -1, 1, 1), dim=8192, heads=64, kv=8, layers=80,
                               vocab=131072, theta=5e5, seq=8192, ffn=28672, head=True)),
])
def test_other_fuji_sizes_match_reference_config_dumps(name, want):
    cfg = fuji.trainer_configs()[name]()
    flat = cfg.to_flat_dict(omit_default_values=set())
    att = "model.decoder.transformer.layer.self_attention.attention."
    assert flat["max_step"] == want["max_step"]
    assert flat["learner.optimizer.args[1].learning_rate"] == want["lr"]
    assert flat["learner.optimizer.args[1].weight_decay"] == 0.1
    assert tuple(flat[f"mesh_shape[{i}]"] for i in range(6)) == want["mesh"]
    assert flat["model.decoder.dim"] == want["dim"] and flat["model.decoder.vocab_size"] == want["vocab"]
    assert flat["model.decoder.transformer.num_layers"] == want["layers"]
    assert flat[att + "num_heads"] == want["heads"]
    assert flat[att + "input_linear.input_linear.num_kv_heads"] == want["kv"]
    assert flat[att + "input_linear.rope_pos_emb_layer.theta"] == want["theta"]
    assert flat["input.source_length"] == want["seq"]
    shapes = _ours(cfg.model, want["layers"])
    assert shapes["decoder/transformer/repeat/layer/feed_forward/linear1_0/weight"] == (want["dim"], want["ffn"])
    assert ("decoder/lm_head/weight" in shapes) == want["head"]


REFERENCE_FUJI_CONFIG_NAMES = """
fuji-1B-v3 fuji-1B-v3-flash fuji-1B-v3-flash-fp8 fuji-1B-v3-flash-fp8-single-host fuji-1B-v3-flash-single-host
fuji-1B-v3-fp8 fuji-1B-v3-fp8-single-host fuji-1B-v3-single-host fuji-1B-v3-tiktoken fuji-1B-v3-tiktoken-flash
fuji-1B-v3-tiktoken-flash-fp8 fuji-1B-v3-tiktoken-flash-fp8-single-host fuji-1B-v3-tiktoken-flash-single-host
fuji-1B-v3-tiktoken-fp8 fuji-1B-v3-tiktoken-fp8-single-host fuji-1B-v3-tiktoken-single-host fuji-3B-v3
fuji-3B-v3-flash fuji-3B-v3-flash-fp8 fuji-3B-v3-flash-fp8-single-host fuji-3B-v3-flash-single-host fuji-3B-v3-fp8
fuji-3B-v3-fp8-single-host fuji-3B-v3-single-host fuji-3B-v3-tiktoken fuji-3B-v3-tiktoken-flash
fuji-3B-v3-tiktoken-flash-fp8 fuji-3B-v3-tiktoken-flash-fp8-single-host fuji-3B-v3-tiktoken-flash-single-host
fuji-3B-v3-tiktoken-fp8 fuji-3B-v3-tiktoken-fp8-single-host fuji-3B-v3-tiktoken-single-host fuji-405B-v3
fuji-405B-v3-flash fuji-405B-v3-flash-fp8 fuji-405B-v3-fp8 fuji-405B-v3-tiktoken fuji-405B-v3-tiktoken-flash
fuji-405B-v3-tiktoken-flash-fp8 fuji-405B-v3-tiktoken-fp8 fuji-70B-v1 fuji-70B-v1-flash fuji-70B-v1-flash-fp8
fuji-70B-v1-fp8 fuji-70B-v2 fuji-70B-v2-flash fuji-70B-v2-flash-fp8 fuji-70B-v2-fp8 fuji-70B-v3 fuji-70B-v3-flash
fuji-70B-v3-flash-fp8 fuji-70B-v3-fp8 fuji-70B-v3-tiktoken fuji-70B-v3-tiktoken-flash fuji-70B-v3-tiktoken-flash-fp8
fuji-70B-v3-tiktoken-fp8 fuji-7B-v1 fuji-7B-v1-flash fuji-7B-v1-flash-fp8 fuji-7B-v1-flash-fp8-single-host
fuji-7B-v1-flash-single-host fuji-7B-v1-fp8 fuji-7B-v1-fp8-single-host fuji-7B-v1-single-host fuji-7B-v2
fuji-7B-v2-flash fuji-7B-v2-flash-fp8 fuji-7B-v2-flash-fp8-single-host fuji-7B-v2-flash-single-host fuji-7B-v2-fp8
fuji-7B-v2-fp8-single-host fuji-7B-v2-single-host fuji-7B-v3 fuji-7B-v3-flash fuji-7B-v3-flash-fp8
fuji-7B-v3-flash-fp8-single-host fuji-7B-v3-flash-single-host fuji-7B-v3-fp8 fuji-7B-v3-fp8-single-host
fuji-7B-v3-single-host fuji-8B-v3-tiktoken fuji-8B-v3-tiktoken-flash fuji-8B-v3-tiktoken-flash-fp8
fuji-8B-v3-tiktoken-flash-fp8-single-host fuji-8B-v3-tiktoken-flash-single-host fuji-8B-v3-tiktoken-fp8
fuji-8B-v3-tiktoken-fp8-single-host fuji-8B-v3-tiktoken-single-host fuji-golden-run-test-v1 fuji-golden-run-test-v2
fuji-golden-run-test-v3 fuji-golden-run-test-v3-tiktoken fuji-test-v1 fuji-test-v1-flash fuji-test-v2
fuji-test-v2-flash fuji-test-v3 fuji-test-v3-flash fuji-test-v3-tiktoken fuji-test-v3-tiktoken-flash
""".split()


def test_fuji_config_names_are_the_reference_set():
    assert sorted(fuji.trainer_configs()) == sorted(REFERENCE_FUJI_CONFIG_NAMES)
    assert len(REFERENCE_FUJI_CONFIG_NAMES) == 100


@pytest.mark.parametrize("name,want", [
    ("fuji-3B-v3-flash", dict(max_step=983040, dim=3072, heads=24, kv=8, layers=28, vocab=131072, ffn=8192, seq=8192)),
    ("fuji-8B-v3-tiktoken-flash", dict(max_step=983040, dim=4096, heads=32, kv=8, layers=32, vocab=128256, ffn=14336, seq=8192)),
    ("fuji-70B-v1-flash", dict(max_step=367001, dim=8192, heads=64, kv=None, layers=80, vocab=32768, ffn=28672, seq=2048)),
    ("fuji-7B-v1-flash", dict(max_step=262144, dim=4096, heads=32, kv=None, layers=32, vocab=32768, ffn=11008, seq=2048)),
    ("fuji-405B-v3-flash", dict(max_step=983040, dim=16384, heads=128, kv=8, layers=126, vocab=131072, ffn=53248, seq=8192)),
])
def test_more_fuji_sizes_match_reference_config_dumps(name, want):
    cfg = fuji.trainer_configs()[name]()
    flat = cfg.to_flat_dict(omit_default_values=set())
    att = "model.decoder.transformer.layer.self_attention.attention."
    assert flat["max_step"] == want["max_step"]
    assert flat["model.decoder.dim"] == want["dim"] and flat["model.decoder.vocab_size"] == want["vocab"]
    assert flat["model.decoder.transformer.num_layers"] == want["layers"]
    assert flat[att + "num_heads"] == want["heads"]
    assert flat.get(att + "input_linear.input_linear.num_kv_heads") == want["kv"]
    assert flat["input.source_length"] == want["seq"]
    shapes = _ours(cfg.model, want["layers"])
    assert shapes["decoder/transformer/repeat/layer/feed_forward/linear2/weight"] == (want["ffn"], want["dim"])


def test_trainer_state_leaf_names_follow_the_reference_checkpoint_layout(tmp_path):
    """``flatten_items(trainer_state)`` names = the tensor names of a checkpoint.  For
    ``chain(clip, chain(scale_by_adam, scale_by_schedule, add_decayed_weights, scale_by_schedule,
    scale))`` the reference stores ``learner/optimizer/1/0/{count,mu/<param>,nu/<param>}``,
    ``learner/optimizer/1/1/count`` and ``learner/optimizer/1/3/count``; stateless links store
    nothing (axlearn/common/state_builder_test.py:797-806, axlearn/common/optimizers.py:584-590)."""
    from axlearn_b200.common import prng
    from tests.helpers import tiny_fuji_trainer_config

    trainer = tiny_fuji_trainer_config(str(tmp_path), max_step=2, save_every_n_steps=100).instantiate(parent=None)
    trainer.init(prng.PRNGKey(0))
    names = [p for p, _ in flatten_items(trainer.trainer_state)]
    params = [n[len("model/"):] for n in names if n.startswith("model/")]
    assert "decoder/transformer/repeat/layer/self_attention/attention/i_proj/i_proj/qkv_proj/weight" in params
    learner = sorted(n for n in names if n.startswith("learner/"))
    want = sorted(["learner/optimizer/1/0/count", "learner/optimizer/1/1/count", "learner/optimizer/1/3/count"]
                  + [f"learner/optimizer/1/0/{m}/{p}" for m in ("mu", "nu") for p in params])
    assert learner == want
    assert "prng_key" in names and len(names) == len(params) + len(want) + 1


def test_envy_switch_base_hyperparameters_match_reference_config_dump():
    cfg = envy.trainer_configs()["envy-Switch-Base"]()
    flat = cfg.to_flat_dict(omit_default_values=set())
    sparse = "model.decoder.transformer.layer.layer[1].feed_forward."
    want = {
        "max_step": 250000, "checkpointer.keep_every_n_steps": 5000,
        "learner.optimizer.args[0].max_norm": 1,
        "learner.optimizer.args[1].b1": 0.9, "learner.optimizer.args[1].b2": 0.95, "learner.optimizer.args[1].eps": 1e-8,
        "learner.optimizer.args[1].learning_rate": 0.01, "learner.optimizer.args[1].weight_decay": 1e-4,
        "learner.optimizer.args[1].update_schedule.alpha": 0.005,
        "learner.optimizer.args[1].update_schedule.warmup_steps": 5000,
        "mesh_shape[2]": 16, "mesh_shape[3]": -1,
        "model.decoder.output_norm.eps": 1e-5,
        "model.decoder.transformer.layer.layer[0].self_attention.attention.input_linear.rope_pos_emb_layer.theta": 5e5,
        "model.decoder.transformer.layer.layer[0].self_attention.attention.query_scale.norm.eps": 1e-5,
        sparse + "gating.train_capacity_factor": 2.0, sparse + "gating.eval_capacity_factor": 2.0,
        sparse + "load_balance_loss_weight": 0.01, sparse + "router_z_loss_weight": 0.0,
        sparse + "num_experts": 128, sparse + "num_groups": 2,
        "model.metrics.metrics['lm'].z_loss_scale": 1e-6,
        "input.source_length": 8192,
    }
    missing = [k for k in want if k not in flat]
    assert not missing, missing
    wrong = {k: (flat[k], v) for k, v in want.items() if flat[k] != v}
    assert not wrong, wrong
    assert flat["input.global_batch_size"] * flat["input.source_length"] == 8 * 2 ** 20
    assert "scale_update_per_param" in str(flat["learner.optimizer.args[1].adam_update_transformation.fn"])


QWEN3_30B_A3B = """
decoder/emb/token_emb/weight 151936,2048
decoder/transformer/repeat/layer/self_attention/norm/scale
decoder/transformer/repeat/layer/self_attention/attention/i_proj/i_proj/qkv_proj/weight 2048,40,128
decoder/transformer/repeat/layer/self_attention/attention/o_proj/weight 2048,32,128
decoder/transformer/repeat/layer/self_attention/attention/scale_query/norm/scale
decoder/transformer/repeat/layer/self_attention/attention/scale_key/norm/scale
decoder/transformer/repeat/layer/feed_forward/gate_weight 2048,128
decoder/transformer/repeat/layer/feed_forward/wo_weight 128,768,2048
decoder/transformer/repeat/layer/feed_forward/wi_0_weight 128,2048,768
decoder/transformer/repeat/layer/feed_forward/wi_1_weight 128,2048,768
decoder/transformer/repeat/layer/feed_forward/norm/scale
decoder/output_norm/scale
decoder/lm_head/weight 151936,2048
"""


def test_qwen3_matches_reference_listing_and_config_dump():
    from axlearn_b200.experiments.text.gpt import qwen

    cfgs = qwen.trainer_configs()
    assert {"qwen3-30B-A3B-bs8m-seq8k", "qwen3-30B-A3B-bs16m-seq32k"} <= set(cfgs)
    cfg = cfgs["qwen3-30B-A3B-bs8m-seq8k"]()
    ours, want = _ours(cfg.model, 48), _golden(QWEN3_30B_A3B)
    assert set(ours) == set(want), sorted(set(ours) ^ set(want))
    for name, shape in want.items():
        if shape is not None:
            assert ours[name] == shape, name
    flat = cfg.to_flat_dict(omit_default_values=set())
    layer = "model.decoder.transformer.layer."
    want_cfg = {
        "max_step": 250000, "learner.optimizer.args[1].learning_rate": 0.01,
        "learner.optimizer.args[1].update_schedule.alpha": 0.005,
        "learner.optimizer.args[1].update_schedule.warmup_steps": 5000,
        "learner.optimizer.args[1].weight_decay": 1e-4,
        "mesh_shape[1]": -1, "mesh_shape[3]": 8,
        "model.decoder.output_norm.eps": 1e-6,
        layer + "feed_forward.gating.num_experts_per_token": 8,
        layer + "feed_forward.hidden_dim": 768,
        layer + "feed_forward.load_balance_loss_weight": 0.001,
        layer + "feed_forward.num_experts": 128,
        layer + "self_attention.attention.hidden_dim": 4096,
        layer + "self_attention.attention.input_linear.input_linear.num_kv_heads": 4,
        layer + "self_attention.attention.input_linear.rope_pos_emb_layer.theta": 1e6,
        layer + "self_attention.attention.query_scale.norm.eps": 1e-6,
        layer + "self_attention.attention.num_heads": 32,
        "model.decoder.transformer.num_layers": 48, "model.decoder.vocab_size": 151936,
        "model.metrics.metrics['lm'].z_loss_scale": 1e-6,
        "input.source_length": 8192,
    }
    missing = [k for k in want_cfg if k not in flat]
    assert not missing, missing
    wrong = {k: (flat[k], v) for k, v in want_cfg.items() if flat[k] != v}
    assert not wrong, wrong
    assert "TopKDropFreeGating" in str(flat[layer + "feed_forward.gating.klass"])
    assert "TransformerFeedForwardDropFreeMoE" in str(flat[layer + "feed_forward.klass"])


RESNET18_WEIGHTS = """
backbone/stem/conv1/weight 7,7,3,64
backbone/stage0/block0/conv1/weight 3,3,64,64
backbone/stage0/block0/conv2/weight 3,3,64,64
backbone/stage0/block1/conv1/weight 3,3,64,64
backbone/stage0/block1/conv2/weight 3,3,64,64
backbone/stage1/block0/conv1/weight 3,3,64,128
backbone/stage1/block0/conv2/weight 3,3,128,128
backbone/stage1/block0/downsample/conv/weight 1,1,64,128
backbone/stage1/block1/conv1/weight 3,3,128,128
backbone/stage1/block1/conv2/weight 3,3,128,128
backbone/stage2/block0/conv1/weight 3,3,128,256
backbone/stage2/block0/conv2/weight 3,3,256,256
backbone/stage2/block0/downsample/conv/weight 1,1,128,256
backbone/stage2/block1/conv1/weight 3,3,256,256
backbone/stage2/block1/conv2/weight 3,3,256,256
backbone/stage3/block0/conv1/weight 3,3,256,512
backbone/stage3/block0/conv2/weight 3,3,512,512
backbone/stage3/block0/downsample/conv/weight 1,1,256,512
backbone/stage3/block1/conv1/weight 3,3,512,512
backbone/stage3/block1/conv2/weight 3,3,512,512
classifier/weight 512,1000
classifier/bias
"""

RESNET50_WEIGHTS = """
backbone/stem/conv1/weight 7,7,3,64
backbone/stage0/block0/conv1/weight 1,1,64,64
backbone/stage0/block0/conv2/weight 3,3,64,64
backbone/stage0/block0/conv3/weight 1,1,64,256
backbone/stage0/block0/downsample/conv/weight 1,1,64,256
backbone/stage0/block1/conv1/weight 1,1,256,64
backbone/stage0/block1/conv2/weight 3,3,64,64
backbone/stage0/block1/conv3/weight 1,1,64,256
backbone/stage0/block2/conv1/weight 1,1,256,64
backbone/stage0/block2/conv2/weight 3,3,64,64
backbone/stage0/block2/conv3/weight 1,1,64,256
backbone/stage1/block0/conv1/weight 1,1,256,128
backbone/stage1/block0/conv2/weight 3,3,128,128
backbone/stage1/block0/conv3/weight 1,1,128,512
backbone/stage1/block0/downsample/conv/weight 1,1,256,512
backbone/stage1/block1/conv1/weight 1,1,512,128
backbone/stage1/block1/conv2/weight 3,3,128,128
backbone/stage1/block1/conv3/weight 1,1,128,512
backbone/stage1/block2/conv1/weight 1,1,512,128
backbone/stage1/block2/conv2/weight 3,3,128,128
backbone/stage1/block2/conv3/weight 1,1,128,512
backbone/stage1/block3/conv1/weight 1,1,512,128
backbone/stage1/block3/conv2/weight 3,3,128,128
backbone/stage1/block3/conv3/weight 1,1,128,512
backbone/stage2/block0/conv1/weight 1,1,512,256
backbone/stage2/block0/conv2/weight 3,3,256,256
backbone/stage2/block0/conv3/weight 1,1,256,1024
backbone/stage2/block0/downsample/conv/weight 1,1,512,1024
backbone/stage2/block1/conv1/weight 1,1,1024,256
backbone/stage2/block1/conv2/weight 3,3,256,256
backbone/stage2/block1/conv3/weight 1,1,256,1024
backbone/stage2/block2/conv1/weight 1,1,1024,256
backbone/stage2/block2/conv2/weight 3,3,256,256
backbone/stage2/block2/conv3/weight 1,1,256,1024
backbone/stage2/block3/conv1/weight 1,1,1024,256
backbone/stage2/block3/conv2/weight 3,3,256,256
backbone/stage2/block3/conv3/weight 1,1,256,1024
backbone/stage2/block4/conv1/weight 1,1,1024,256
backbone/stage2/block4/conv2/weight 3,3,256,256
backbone/stage2/block4/conv3/weight 1,1,256,1024
backbone/stage2/block5/conv1/weight 1,1,1024,256
backbone/stage2/block5/conv2/weight 3,3,256,256
backbone/stage2/block5/conv3/weight 1,1,256,1024
backbone/stage3/block0/conv1/weight 1,1,1024,512
backbone/stage3/block0/conv2/weight 3,3,512,512
backbone/stage3/block0/conv3/weight 1,1,512,2048
backbone/stage3/block0/downsample/conv/weight 1,1,1024,2048
backbone/stage3/block1/conv1/weight 1,1,2048,512
backbone/stage3/block1/conv2/weight 3,3,512,512
backbone/stage3/block1/conv3/weight 1,1,512,2048
backbone/stage3/block2/conv1/weight 1,1,2048,512
backbone/stage3/block2/conv2/weight 3,3,512,512
backbone/stage3/block2/conv3/weight 1,1,512,2048
classifier/weight 2048,1000
classifier/bias
"""


@pytest.mark.parametrize("name,listing", [("resnet18", RESNET18_WEIGHTS), ("resnet50", RESNET50_WEIGHTS)])
def test_resnet_matches_reference_listing(name, listing):
    """Convolution / classifier weights by name and shape; every convolution ``convN`` has its
    ``normN`` sibling (``downsample/conv`` has ``downsample/norm``) with scale, bias and the two
    moving statistics, as in the reference's ``ResNet-18_init.txt`` / ``ResNet-50_init.txt``."""
    from axlearn_b200.vision.image_classification import ImageClassificationModel
    from axlearn_b200.vision.resnet import named_resnet_config

    model = ImageClassificationModel.default_config().set(
        name="model", backbone=named_resnet_config(name), num_classes=1000).instantiate(parent=None)
    specs = dict(flatten_items(model.create_parameter_specs_recursively(), is_leaf=lambda x: hasattr(x, "mesh_axes")))
    want = _golden(listing)
    ours_weights = {p: tuple(s.shape) for p, s in specs.items() if "norm" not in p}
    assert set(ours_weights) == set(want), sorted(set(ours_weights) ^ set(want))[:10]
    for path, shape in want.items():
        if shape is not None:
            assert ours_weights[path] == shape, path
    for path in want:
        if path.endswith("/weight") and "conv" in path.rsplit("/", 2)[-2]:
            norm = path.rsplit("/", 2)[0] + "/" + path.rsplit("/", 2)[-2].replace("conv", "norm")
            for leaf in ("scale", "bias", "moving_mean", "moving_variance"):
                assert f"{norm}/{leaf}" in specs, f"{norm}/{leaf}"


CONFORMER_TEST_CTC = """
encoder/feature/subsampler/conv1/weight 3,3,1,4
encoder/feature/subsampler/conv1/bias
encoder/feature/subsampler/conv2/weight 3,3,4,4
encoder/feature/subsampler/conv2/bias
encoder/context/input_linear/weight 80,4
encoder/context/input_linear/bias
encoder/context/context/repeat/layer/ff_start/norm/scale
encoder/context/context/repeat/layer/ff_start/norm/bias
encoder/context/context/repeat/layer/ff_start/linear1/weight 4,16
encoder/context/context/repeat/layer/ff_start/linear1/bias
encoder/context/context/repeat/layer/ff_start/linear2/weight 16,4
encoder/context/context/repeat/layer/ff_start/linear2/bias
encoder/context/context/repeat/layer/ff_end/norm/scale
encoder/context/context/repeat/layer/ff_end/norm/bias
encoder/context/context/repeat/layer/ff_end/linear1/weight 4,16
encoder/context/context/repeat/layer/ff_end/linear1/bias
encoder/context/context/repeat/layer/ff_end/linear2/weight 16,4
encoder/context/context/repeat/layer/ff_end/linear2/bias
encoder/context/context/repeat/layer/self_attention/norm/scale
encoder/context/context/repeat/layer/self_attention/norm/bias
encoder/context/context/repeat/layer/self_attention/attention/u_bias
encoder/context/context/repeat/layer/self_attention/attention/v_bias
encoder/context/context/repeat/layer/self_attention/attention/i_proj/qkv_proj/weight 4,2,2
encoder/context/context/repeat/layer/self_attention/attention/i_proj/qkv_proj/bias
encoder/context/context/repeat/layer/self_attention/attention/o_proj/weight 4,2,2
encoder/context/context/repeat/layer/self_attention/attention/o_proj/bias
encoder/context/context/repeat/layer/self_attention/attention/scale_query/per_dim_scale/param
encoder/context/context/repeat/layer/self_attention/attention/r_proj/weight 4,2,2
encoder/context/context/repeat/layer/lconv/linear1_norm/scale
encoder/context/context/repeat/layer/lconv/linear1_norm/bias
encoder/context/context/repeat/layer/lconv/linear1_0/weight 4,4
encoder/context/context/repeat/layer/lconv/linear1_0/bias
encoder/context/context/repeat/layer/lconv/linear1_1/weight 4,4
encoder/context/context/repeat/layer/lconv/linear1_1/bias
encoder/context/context/repeat/layer/lconv/conv/weight 32,1,4
encoder/context/context/repeat/layer/lconv/conv_norm/scale
encoder/context/context/repeat/layer/lconv/conv_norm/bias
encoder/context/context/repeat/layer/lconv/conv_norm/moving_mean
encoder/context/context/repeat/layer/lconv/conv_norm/moving_variance
encoder/context/context/repeat/layer/lconv/linear2/weight 4,4
encoder/context/context/repeat/layer/lconv/linear2/bias
encoder/context/context/repeat/layer/norm/scale
encoder/context/context/repeat/layer/norm/bias
decoder/lm_head/weight
decoder/lm_head/bias
"""


def test_conformer_ctc_model_matches_reference_listing():
    """Parameter names (and the shapes the listing gives) of the ``conformer-test-ctc`` speech
    recogniser: log-mel features -> 2 x stride-2 convolutions -> input projection -> stacked
    conformer layers with Transformer-XL attention -> CTC head."""
    from axlearn_b200.audio.asr import ASREncoder, ASRModel, CTCDecoderModel, SpeechFeatureLayer
    from axlearn_b200.audio.frontend import LogMelFrontend
    from axlearn_b200.audio.subsamplers import ConvSubSampler

    dim, heads, filters, layers, vocab = 4, 2, 80, 2, 1024
    feature = SpeechFeatureLayer.default_config().set(
        output_dim=dim, frontend=LogMelFrontend.default_config().set(
            num_filters=filters, sample_rate=16000, frame_size_ms=25, hop_size_ms=10),
        subsampler=ConvSubSampler.default_config())
    enc = ASREncoder.default_config().set(dim=dim, feature=feature, feature_dim=filters // 4 * dim)
    enc.context.context.set(num_layers=layers)
    enc.context.context.layer.set(num_heads=heads)
    model = ASRModel.default_config().set(
        name="model", encoder=enc, decoder=CTCDecoderModel.default_config().set(input_dim=dim, vocab_size=vocab)
    ).instantiate(parent=None)
    specs = dict(flatten_items(model.create_parameter_specs_recursively(), is_leaf=lambda x: hasattr(x, "mesh_axes")))
    want = _golden(CONFORMER_TEST_CTC)
    assert set(specs) == set(want), sorted(set(specs) ^ set(want))
    for path, shape in want.items():
        if shape is None:
            continue
        ours = tuple(specs[path].shape)
        if "/repeat/" in path:
            assert ours[0] == layers
            ours = ours[1:]
        if path.endswith("qkv_proj/weight"):
            assert ours[0] == 3
            ours = ours[1:]
        assert ours == shape, path
