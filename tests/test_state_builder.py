"""State builders: warm-starting a trainer from another run's checkpoint, scope conversion."""

import os

import torch

from axlearn_b200.common import prng, state_builder
from axlearn_b200.common.checkpointer import latest_checkpoint_path
from tests.helpers import tiny_fuji_trainer_config

KW = dict(save_every_n_steps=2, hidden=32, heads=2, ffn=64, vocab=64, seq=16, batch=4)


def _trained(tmp_path, layers=2):
    cfg = tiny_fuji_trainer_config(tmp_path / "src", max_step=2, layers=layers, **KW)
    trainer = cfg.instantiate(parent=None)
    trainer.run(prng.PRNGKey(0))
    return trainer, latest_checkpoint_path(os.path.join(str(tmp_path / "src"), "checkpoints"))


def test_tensorstore_builder_warm_starts_model_params(tmp_path):
    src, ckpt = _trained(tmp_path)
    cfg = tiny_fuji_trainer_config(tmp_path / "dst", max_step=2, layers=2, **KW)
    cfg.init_state_builder = state_builder.TensorStoreStateStorageBuilder.default_config().set(
        dir=ckpt, include=r"model/.*")
    dst = cfg.instantiate(parent=None)
    dst.init(prng.PRNGKey(123))          # a different seed: everything must come from the checkpoint
    a = src.trainer_state["model"]["decoder"]["transformer"]["repeat"]["layer"]["feed_forward"]["linear2"]["weight"]
    b = dst.trainer_state["model"]["decoder"]["transformer"]["repeat"]["layer"]["feed_forward"]["linear2"]["weight"]
    assert torch.equal(a, b)
    # The optimizer state is fresh.
    assert int(dst.step) == 0


def test_scope_converter_loads_only_the_named_subtree(tmp_path):
    src, ckpt = _trained(tmp_path)
    cfg = tiny_fuji_trainer_config(tmp_path / "dst", max_step=2, layers=2, **KW)
    cfg.init_state_builder = state_builder.RestoreAndConvertBuilder.default_config().set(
        builder=state_builder.TensorStoreStateStorageBuilder.default_config().set(dir=ckpt),
        converter=state_builder.ModelStateScopeConverter.default_config().set(scope="decoder/emb"))
    dst = cfg.instantiate(parent=None)
    dst.init(prng.PRNGKey(123))
    emb = lambda t: t.trainer_state["model"]["decoder"]["emb"]["token_emb"]["weight"]
    ffn = lambda t: t.trainer_state["model"]["decoder"]["transformer"]["repeat"]["layer"]["feed_forward"]["linear2"]["weight"]
    assert torch.equal(emb(src), emb(dst))
    assert not torch.equal(ffn(src), ffn(dst))     # outside the scope: freshly initialised


def test_chain_and_weight_modifier():
    state = state_builder.Builder.State(
        step=0, trainer_state={"model": {"a": {"weight": torch.ones(2, 2)}, "b": {"weight": torch.ones(2)}}},
        built_keys=set())
    mod = state_builder.SimpleWeightModifierBuilder.default_config().set(
        path_regex=r"a/.*", modify=lambda path, t: t * 3)
    chain = state_builder.ChainBuilder.default_config().set(name="c", builders=[mod, mod]).instantiate(parent=None)
    out = chain(state)
    assert torch.equal(out.trainer_state["model"]["a"]["weight"], torch.full((2, 2), 9.0))
    assert torch.equal(out.trainer_state["model"]["b"]["weight"], torch.ones(2))
    assert isinstance(state_builder.get_builder_config("/x/checkpoints/step_00000010").set(name="b").instantiate(parent=None),
                      state_builder.TensorStoreStateStorageBuilder)
