"""Hugging Face Llama <-> Fuji parameter conversion: logits must agree with ``transformers``."""

import pytest
import torch

from axlearn_b200.common import prng
from axlearn_b200.common.module import functional
from axlearn_b200.common.param_converter import fuji_to_llama_hf, llama_hf_to_fuji
from axlearn_b200.common.utils import flatten_items
from axlearn_b200.experiments.text.gpt import fuji

transformers = pytest.importorskip("transformers")


def _hf_model(num_kv_heads, tie):
    cfg = transformers.LlamaConfig(
        vocab_size=96, hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4,
        num_key_value_heads=num_kv_heads, rms_norm_eps=1e-5, rope_theta=10000.0, tie_word_embeddings=tie,
        attention_bias=False, mlp_bias=False, max_position_embeddings=64)
    torch.manual_seed(0)
    model = transformers.LlamaForCausalLM(cfg).eval()
    with torch.no_grad():
        for p in model.parameters():          # norms away from 1 so that a mix-up would show
            if p.dim() == 1:
                p.add_(torch.randn_like(p) * 0.1)
    return model


@pytest.mark.parametrize("num_kv_heads,grouped,tie", [(4, False, False), (2, True, False), (2, True, True)])
def test_llama_logits_match_transformers(num_kv_heads, grouped, tie):
    hf = _hf_model(num_kv_heads, tie)
    ours_cfg = fuji.model_config(
        num_layers=2, hidden_dim=64, num_heads=4, num_kv_heads=num_kv_heads if grouped else None, vocab_size=96,
        rope_theta=1e4, shared_lm_head=tie, ffn_dim=128).set(name="model")
    model = ours_cfg.instantiate(parent=None)
    params = llama_hf_to_fuji(hf.state_dict(), num_layers=2, num_heads=4,
                              num_kv_heads=num_kv_heads if grouped else None)
    # Same tree (names and shapes) as a fresh initialisation of the model.
    init = model.initialize_parameters_recursively(prng.PRNGKey(0), device="cpu")
    want = {p: tuple(t.shape) for p, t in flatten_items(init)}
    got = {p: tuple(t.shape) for p, t in flatten_items(params)}
    assert got == want
    ids = torch.randint(0, 96, (2, 17))
    with torch.no_grad():
        ref = hf(input_ids=ids).logits
        out, _ = functional(model, prng.PRNGKey(1), params, dict(input_batch={"input_ids": ids}),
                            is_training=False, method="predict")
        if "logits" not in out:
            logits, _ = functional(model, prng.PRNGKey(1), params, dict(predict_outputs=out), is_training=False,
                                   method="compute_logits")
        else:
            logits = out["logits"]
    torch.testing.assert_close(logits, ref, rtol=2e-4, atol=2e-4)
    # And back.
    back = fuji_to_llama_hf(params, num_heads=4, num_kv_heads=num_kv_heads if grouped else None)
    for name, t in hf.state_dict().items():
        torch.testing.assert_close(back[name], t)
