"""Selective rematerialisation: policies decide what a replayed layer keeps, never its gradients."""

import torch

from axlearn_b200.common import prng, remat
from axlearn_b200.common.attention import RematRegexSavePatterns, build_remat_spec
from axlearn_b200.common.base_layer import RematSpec, nothing_saveable
from axlearn_b200.common.config import config_for_function
from axlearn_b200.common.module import functional
from axlearn_b200.common.utils import flatten_items
from axlearn_b200.experiments.text.gpt import fuji


def _model(remat_spec):
    cfg = fuji.model_config(num_layers=3, hidden_dim=64, num_heads=4, num_kv_heads=2, vocab_size=128,
                            rope_theta=1e4, shared_lm_head=True, ffn_dim=128)
    cfg.decoder.transformer.layer.remat_spec = remat_spec
    cfg.name = "model"
    model = cfg.instantiate(parent=None)
    params = model.initialize_parameters_recursively(prng.PRNGKey(0))
    return model, params


def _loss_and_grads(remat_spec, monkeypatch=None):
    model, params = _model(remat_spec)
    leaves = [t.requires_grad_() for _, t in flatten_items(params)]
    torch.manual_seed(0)
    ids = torch.randint(0, 128, (2, 17))
    batch = {"input_ids": ids[:, :-1], "target_labels": ids[:, 1:]}
    (loss, _), _ = functional(model, prng.PRNGKey(1), params, [batch], is_training=True, method="forward")
    loss.backward()
    return loss.detach(), [t.grad.clone() for t in leaves]


def test_policy_vocabulary():
    pol = remat.save_only_these_names_regex(RematRegexSavePatterns.NATIVE_ATTENTION.value)
    assert pol("MultiheadAttention.q_proj") == "save"
    assert pol("GroupedQueryAttention.context") == "save"
    assert pol("TransformerFeedForwardLayer.linear1_0") is None
    both = remat.save_and_offload_only_these_names_regex(
        names_which_can_be_saved=".*o_proj", names_which_can_be_offloaded=".*linear1_[01]")
    assert both("X.o_proj") == "save" and both("Y.linear1_1") == "offload" and both("Y.linear2") is None
    assert remat.as_policy(nothing_saveable) is None
    assert remat.as_policy(remat.dots_saveable()).dots == "save"
    assert remat.as_policy(remat.offload_dots_saveable()).dots == "offload"
    spec = build_remat_spec(fuji.model_config(
        num_layers=2, hidden_dim=64, num_heads=4, num_kv_heads=None, vocab_size=128, rope_theta=1e4,
        shared_lm_head=True, ffn_dim=128).decoder.transformer)
    assert spec.selective_policy()("MultiheadAttention.v_proj") == "save"


def test_policies_do_not_change_loss_or_gradients():
    base_loss, base_grads = _loss_and_grads(None)
    specs = {
        "full": RematSpec(policy=nothing_saveable),
        "default": RematSpec(policy=config_for_function(remat.save_only_these_names_regex).set(
            pattern=RematRegexSavePatterns.NATIVE_ATTENTION.value)),
        "ffn_offload": RematSpec(policy=remat.save_and_offload_only_these_names_regex(
            names_which_can_be_saved=RematRegexSavePatterns.NATIVE_ATTENTION.value,
            names_which_can_be_offloaded=RematRegexSavePatterns.FEED_FORWARD.value)),
        "dots": RematSpec(policy=remat.dots_saveable()),
    }
    for name, spec in specs.items():
        loss, grads = _loss_and_grads(spec)
        assert torch.equal(loss, base_loss), name
        for a, b in zip(grads, base_grads):
            assert torch.allclose(a, b, atol=1e-6, rtol=1e-5), name


def test_replay_skips_what_the_policy_kept(monkeypatch):
    """Counts projection products executed: full remat replays all of them, the default policy
    skips the replay of the q/k/v and output projections, ``dots_saveable`` skips every one."""
    from axlearn_b200.ops import dispatch

    calls = {"n": 0}
    real = dispatch._linear_impl  # pylint: disable=protected-access

    def counting(x, w):
        calls["n"] += 1
        return real(x, w)

    monkeypatch.setattr(dispatch, "_linear_impl", counting)

    def count(spec):
        calls["n"] = 0
        _loss_and_grads(spec)
        return calls["n"]

    none = count(None)
    full = count(RematSpec(policy=nothing_saveable))
    default = count(RematSpec(policy=remat.save_only_these_names_regex(RematRegexSavePatterns.NATIVE_ATTENTION.value)))
    dots = count(RematSpec(policy=remat.dots_saveable()))
    per_layer = (none - 1) // 3 if (none - 1) % 3 == 0 else None  # projections per layer (+ the LM head once)
    assert full > none  # the replay runs every projection a second time
    assert none <= dots < default < full
    assert dots == none  # nothing is replayed
    if per_layer is not None:
        # q/k/v (one fused product) and the output projection are not replayed.
        assert full - default == 3 * 2


def test_offloaded_tensors_round_trip():
    stash = remat.LayerStash(remat.save_and_offload_only_these_names_regex(names_which_can_be_offloaded=".*ctx"))

    class Owner:
        pass

    t = torch.arange(12.0).reshape(3, 4)
    with remat.recording(stash), remat.tagged(Owner(), "ctx"):
        (out,), replayed = remat.operator_outputs(lambda: (t * 2,), is_dot=False)
    assert not replayed and torch.equal(out, t * 2)
    with remat.replaying(stash), remat.tagged(Owner(), "ctx"):
        (again,), replayed = remat.operator_outputs(lambda: (_ for _ in ()).throw(AssertionError("recomputed")),
                                                     is_dot=False)
    assert replayed and torch.equal(again, t * 2)
    stash.clear()
