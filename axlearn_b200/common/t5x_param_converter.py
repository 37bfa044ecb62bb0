"""T5X (Flax) parameter trees -> this framework's T5 encoder-decoder parameters.

Parity target: axlearn/common/t5x_param_converter.py (``parameters_from_t5x_encoder_decoder`` :416
and its per-layer helpers).  A T5X ``network.Transformer`` checkpoint is a nested dict

    token_embedder/embedding [V, D]
    encoder/layers_{i}/{attention/{query,key,value,out}/kernel, pre_attention_layer_norm/scale,
                        mlp/{wi_0,wi_1,wo}/kernel, pre_mlp_layer_norm/scale}
    encoder/{relpos_bias/rel_embedding [N, buckets], encoder_norm/scale}
    decoder/layers_{i}/{self_attention, pre_self_attention_layer_norm, encoder_decoder_attention,
                        pre_cross_attention_layer_norm, mlp, pre_mlp_layer_norm}
    decoder/{relpos_bias/rel_embedding, decoder_norm/scale, logits_dense/kernel [D, V]}

with kernels stored ``[in, out]``.  T5X folds the ``1 / sqrt(head_dim)`` of the attention logits into
the initialisation of the query kernel; this framework divides the logits explicitly, so query
kernels are multiplied by ``sqrt(head_dim)`` on the way in.  The conversion goes through the
Hugging Face naming (``t5x_to_hf_state_dict``), whose own converter
(``param_converter.t5_hf_to_encoder_decoder``) is checked against ``transformers``.
"""

from __future__ import annotations

from typing import Any, Mapping

import numpy as np
import torch

from axlearn_b200.common.param_converter import t5_hf_to_encoder_decoder

Tensor = torch.Tensor

_ATTENTION = {"query": "q", "key": "k", "value": "v", "out": "o"}
_MLP = ("wi_0", "wi_1", "wo")


def _t(x: Any) -> Tensor:
    return x if isinstance(x, Tensor) else torch.from_numpy(np.asarray(x))


def _only(src: Mapping, allowed: set, where: str) -> None:
    extra = set(src) - allowed
    if extra:
        raise ValueError(f"Unsupported layer(s) under {where}: {sorted(extra)}")


def _attention(src: Mapping, prefix: str, out: dict) -> None:
    _only(src, set(_ATTENTION), prefix)
    for name, short in _ATTENTION.items():
        _only(src[name], {"kernel"}, f"{prefix}{name}")
        out[f"{prefix}{short}.weight"] = _t(src[name]["kernel"]).t().contiguous()       # [in, out] -> [out, in]


def _mlp(src: Mapping, prefix: str, out: dict) -> None:
    _only(src, set(_MLP), prefix)
    for name in _MLP:
        out[f"{prefix}{name}.weight"] = _t(src[name]["kernel"]).t().contiguous()


def _norm(src: Mapping, key: str, out: dict) -> None:
    _only(src, {"scale"}, key)
    out[key] = _t(src["scale"])


def _stack(src: Mapping, side: str, out: dict) -> int:
    """Encoder (``side = "encoder"``) or decoder stack; returns its number of layers."""
    layers = {}
    for name, params in src.items():
        if name.startswith("layers_"):
            layers[int(name.split("_")[-1])] = params
        elif name == f"{side}_norm":
            _norm(params, f"{side}.final_layer_norm.weight", out)
        elif name == "relpos_bias":
            _only(params, {"rel_embedding"}, f"{side}/relpos_bias")
            out[f"{side}.block.0.layer.0.SelfAttention.relative_attention_bias.weight"] = \
                _t(params["rel_embedding"]).t().contiguous()                            # [N, buckets] -> [buckets, N]
        elif name == "logits_dense" and side == "decoder":
            _only(params, {"kernel"}, "decoder/logits_dense")
            out["lm_head.weight"] = _t(params["kernel"]).t().contiguous()
        else:
            raise ValueError(f"Unsupported layer: {side}/{name}")
    if sorted(layers) != list(range(len(layers))):
        raise ValueError(f"{side} layers are not numbered 0..{len(layers) - 1}: {sorted(layers)}")
    for i, layer in layers.items():
        p = f"{side}.block.{i}.layer."
        if side == "encoder":
            _only(layer, {"attention", "pre_attention_layer_norm", "mlp", "pre_mlp_layer_norm"}, f"encoder/layers_{i}")
            _attention(layer["attention"], p + "0.SelfAttention.", out)
            _norm(layer["pre_attention_layer_norm"], p + "0.layer_norm.weight", out)
            _mlp(layer["mlp"], p + "1.DenseReluDense.", out)
            _norm(layer["pre_mlp_layer_norm"], p + "1.layer_norm.weight", out)
        else:
            _only(layer, {"self_attention", "pre_self_attention_layer_norm", "encoder_decoder_attention",
                          "pre_cross_attention_layer_norm", "mlp", "pre_mlp_layer_norm"}, f"decoder/layers_{i}")
            _attention(layer["self_attention"], p + "0.SelfAttention.", out)
            _norm(layer["pre_self_attention_layer_norm"], p + "0.layer_norm.weight", out)
            _attention(layer["encoder_decoder_attention"], p + "1.EncDecAttention.", out)
            _norm(layer["pre_cross_attention_layer_norm"], p + "1.layer_norm.weight", out)
            _mlp(layer["mlp"], p + "2.DenseReluDense.", out)
            _norm(layer["pre_mlp_layer_norm"], p + "2.layer_norm.weight", out)
    return len(layers)


def t5x_to_hf_state_dict(src: Mapping) -> tuple:
    """``(state_dict under T5ForConditionalGeneration's names, encoder layers, decoder layers)``."""
    out: dict = {}
    n_enc = n_dec = 0
    for name, params in src.items():
        if name == "token_embedder":
            _only(params, {"embedding"}, "token_embedder")
            out["shared.weight"] = _t(params["embedding"])
        elif name == "encoder":
            n_enc = _stack(params, "encoder", out)
        elif name == "decoder":
            n_dec = _stack(params, "decoder", out)
        else:
            raise ValueError(f"Unsupported layer: {name}")
    if "lm_head.weight" not in out and "shared.weight" in out:
        out["lm_head.weight"] = out["shared.weight"]          # tied output embedding
    return out, n_enc, n_dec


def parameters_from_t5x_encoder_decoder(src: Mapping, *, num_heads: int) -> dict:
    """T5X ``network.Transformer`` parameters -> the tree of ``t5.t5_encoder_decoder_config``."""
    state_dict, n_enc, n_dec = t5x_to_hf_state_dict(src)
    if n_enc == 0 or n_dec == 0:
        raise ValueError("the source tree needs both an encoder and a decoder")
    return t5_hf_to_encoder_decoder(state_dict, num_heads=num_heads, num_encoder_layers=n_enc, num_decoder_layers=n_dec)
