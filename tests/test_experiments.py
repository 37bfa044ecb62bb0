"""Named experiment configs instantiate, have the documented shapes and take a training step."""

import pytest
import torch

from axlearn_b200.common import prng
from axlearn_b200.common.utils import flatten_items
from axlearn_b200.experiments.text.gpt import envy, fuji, gala, honeycrisp, qwen


def _param_shapes(model_cfg):
    model = model_cfg.clone(name="model").instantiate(parent=None)
    specs = model.create_parameter_specs_recursively()
    return {p: tuple(s.shape) for p, s in flatten_items(specs, is_leaf=lambda x: hasattr(x, "mesh_axes"))}


def test_honeycrisp_3b_shapes():
    kw = honeycrisp.get_trainer_kwargs("3B")
    shapes = _param_shapes(kw["model_cfg"])
    layer = "decoder/transformer/repeat/layer/"
    assert shapes[layer + "self_attention/attention/i_proj/i_proj/qkv_proj/weight"] == (26, 3072, 24 + 2 * 8, 128)
    assert shapes[layer + "feed_forward/linear1_0/weight"] == (26, 3072, 8064)
    assert shapes[layer + "self_attention/attention/scale_query/norm/scale"] == (26, 128)
    assert shapes["decoder/emb/token_emb/weight"] == (48 * 1024, 3072)
    assert not any(p.startswith("decoder/lm_head") for p in shapes)        # tied head
    total = sum(torch.Size(s).numel() for s in shapes.values())
    assert 2.5e9 < total < 3.5e9


def test_gala_sizes_and_structures():
    shapes = _param_shapes(gala.get_trainer_kwargs("7B")["model_cfg"])
    layer = "decoder/transformer/repeat/layer/"
    assert shapes[layer + "self_attention/attention/i_proj/i_proj/qkv_proj/weight"] == (32, 3, 4096, 32, 128)
    assert shapes[layer + "feed_forward/linear2/weight"] == (32, 11008, 4096)
    hybrid = _param_shapes(gala.get_trainer_kwargs("85M", norm_structure="hybridnorm")["model_cfg"])
    assert layer + "feed_forward/prenorm/scale" in hybrid and layer + "feed_forward/postnorm/scale" in hybrid
    alibi = gala.model_config(num_layers=1, hidden_dim=8, num_heads=2, vocab_size=8, position_encoding="alibi")
    assert alibi.decoder.attention_mask.num_heads == 2
    assert set(gala.trainer_configs()) >= {"gala-85M", "gala-7B-hybridnorm-alibi", "gala-1B-hybridnorm-alibi-flash"}
    assert "gala-1B-hybridnorm-alibi" not in gala.trainer_configs()


@pytest.mark.parametrize("name,module", [("honeycrisp-test", honeycrisp), ("gala-test", gala)])
def test_test_sized_configs_train(tmp_path, name, module):
    cfg = module.trainer_configs()[name]()
    cfg.dir = str(tmp_path)
    cfg.device = "cpu"
    cfg.train_dtype = None
    cfg.max_step = 3
    trainer = cfg.instantiate(parent=None)
    trainer.init(prng.PRNGKey(0))
    batch = next(iter(trainer.input.dataset()))
    losses = [trainer.train_step(batch)["loss"].item() for _ in range(12)]
    assert all(torch.isfinite(torch.tensor(losses))) and losses[-1] < losses[0]
    # mup-simple: the update transformation sits inside the AdaStar chain.
    state = trainer.trainer_state["learner"]["optimizer"]
    assert state is not None


def test_all_families_list_their_configs():
    names = set()
    for module in (fuji, envy, qwen, honeycrisp, gala):
        names |= set(module.trainer_configs())
    assert {"envy-Mixtral-8x7B", "qwen3-30B-A3B-bs8m-seq8k", "honeycrisp-3B", "gala-1B"} <= names
    assert any(n.startswith("fuji-7B") for n in names)


def test_gspmd_pipeline_configs(tmp_path):
    from axlearn_b200.experiments.text.gpt import gspmd

    cfgs = gspmd.trainer_configs()
    shapes = _param_shapes(cfgs["gspmd-16B-2x16x8"]().model)
    stage = "decoder/transformer/pipeline/layer/"
    key = next(p for p in shapes if p.startswith(stage) and p.endswith("linear1/weight"))
    assert shapes[key] == (2, 4096, 16384)                                          # [stages, D, 4D]
    assert sum(p.endswith("linear1/weight") for p in shapes) == 32               # layers per stage
    total = sum(torch.Size(s).numel() for s in shapes.values())
    assert 12e9 < total < 18e9
    cfg = cfgs["gspmd-test"]()
    cfg.dir, cfg.device, cfg.train_dtype = str(tmp_path), "cpu", None
    trainer = cfg.instantiate(parent=None)
    trainer.init(prng.PRNGKey(0))
    batch = next(iter(trainer.input.dataset()))
    losses = [trainer.train_step(batch)["loss"].item() for _ in range(10)]
    assert losses[-1] < losses[0]
