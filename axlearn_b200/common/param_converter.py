"""Converting parameters between this framework's layout and Hugging Face checkpoints.

Parity target in the reference: axlearn/common/param_converter.py (torch / Hugging Face <->
AXLearn parameter trees).  Covered here: Llama-family causal LMs (Llama 2 / 3, Mistral-style
dense models) <-> the Fuji layout, both directions.

Layout differences that the conversion handles:

* Linear weights are ``[in, out]`` here and ``[out, in]`` in torch.
* The attention projections are fused and head-shaped: ``qkv_proj/weight`` is ``[3, D, N, H]``
  (multi-head) or ``[D, N + 2 * Nkv, H]`` (grouped-query); ``o_proj/weight`` is ``[D, N, H]``.
* Layers are stacked on a leading ``[L]`` dim (``RepeatedTransformerLayer``).
* Rotary embedding convention: Hugging Face rotates the two *halves* of a head
  (``x[i], x[i + H/2]``), this framework rotates *adjacent pairs* (``x[2i], x[2i + 1]``).  The
  per-head output features of the q and k projections are permuted accordingly; attention
  scores are invariant to a permutation applied to q and k alike, so logits match.
"""

from __future__ import annotations

from typing import Any, Mapping, Optional

import torch

Tensor = torch.Tensor


def _halves_to_pairs(w: Tensor) -> Tensor:
    """Last dim ``H`` from [first half | second half] order to interleaved pairs."""
    h = w.shape[-1]
    return torch.stack([w[..., : h // 2], w[..., h // 2:]], dim=-1).reshape(*w.shape[:-1], h)


def _pairs_to_halves(w: Tensor) -> Tensor:
    h = w.shape[-1]
    pairs = w.reshape(*w.shape[:-1], h // 2, 2)
    return torch.cat([pairs[..., 0], pairs[..., 1]], dim=-1)


def llama_hf_to_fuji(state_dict: Mapping[str, Tensor], *, num_layers: int, num_heads: int,
                     num_kv_heads: Optional[int] = None, dtype: Optional[torch.dtype] = None) -> dict:
    """``LlamaForCausalLM.state_dict()`` -> the ``model`` parameter tree of a Fuji-style
    ``causal_lm.Model`` (fused QKV, stacked layers).  ``num_kv_heads=None`` selects the
    multi-head layout ``[3, D, N, H]``; a number selects the grouped layout (also when it equals
    ``num_heads``).  A tied head (no ``lm_head.weight``) yields no ``lm_head`` entry."""
    sd = {k: (v if dtype is None else v.to(dtype)) for k, v in state_dict.items()}
    emb = sd["model.embed_tokens.weight"]
    d = emb.shape[1]
    h = d // num_heads if "model.layers.0.self_attn.q_proj.weight" not in sd else (
        sd["model.layers.0.self_attn.q_proj.weight"].shape[0] // num_heads)
    nkv = num_kv_heads or num_heads

    def per_layer(fn):
        return torch.stack([fn(i) for i in range(num_layers)], dim=0)

    def heads(name: str, i: int, n: int, rotary: bool) -> Tensor:
        w = sd[f"model.layers.{i}.self_attn.{name}.weight"]          # [n * H, D]
        w = w.t().reshape(d, n, h)                                     # [D, n, H]
        return _halves_to_pairs(w) if rotary else w

    def qkv(i: int) -> Tensor:
        q, k, v = heads("q_proj", i, num_heads, True), heads("k_proj", i, nkv, True), heads("v_proj", i, nkv, False)
        if num_kv_heads is None:
            return torch.stack([q, k, v], dim=0)                       # [3, D, N, H]
        return torch.cat([q, k, v], dim=1)                             # [D, N + 2 Nkv, H]

    def o_proj(i: int) -> Tensor:
        w = sd[f"model.layers.{i}.self_attn.o_proj.weight"]            # [D, N * H]
        return w.reshape(d, num_heads, h)

    layer = {
        "self_attention": {
            "norm": {"scale": per_layer(lambda i: sd[f"model.layers.{i}.input_layernorm.weight"])},
            "attention": {
                "i_proj": {"i_proj": {"qkv_proj": {"weight": per_layer(qkv)}}},
                "o_proj": {"weight": per_layer(o_proj)},
            },
        },
        "feed_forward": {
            "norm": {"scale": per_layer(lambda i: sd[f"model.layers.{i}.post_attention_layernorm.weight"])},
            "linear1_0": {"weight": per_layer(lambda i: sd[f"model.layers.{i}.mlp.gate_proj.weight"].t())},
            "linear1_1": {"weight": per_layer(lambda i: sd[f"model.layers.{i}.mlp.up_proj.weight"].t())},
            "linear2": {"weight": per_layer(lambda i: sd[f"model.layers.{i}.mlp.down_proj.weight"].t())},
        },
    }
    decoder: dict[str, Any] = {
        "emb": {"token_emb": {"weight": emb}},
        "transformer": {"repeat": {"layer": layer}},
        "output_norm": {"scale": sd["model.norm.weight"]},
    }
    if "lm_head.weight" in sd and sd["lm_head.weight"].data_ptr() != emb.data_ptr():
        decoder["lm_head"] = {"weight": sd["lm_head.weight"]}
    return {"decoder": _contiguous(decoder)}


def fuji_to_llama_hf(params: Mapping[str, Any], *, num_heads: int, num_kv_heads: Optional[int] = None) -> dict:
    """The inverse of ``llama_hf_to_fuji``: a ``state_dict`` loadable into ``LlamaForCausalLM``."""
    dec = params["decoder"]
    layer = dec["transformer"]["repeat"]["layer"]
    att = layer["self_attention"]["attention"]
    qkv = att["i_proj"]["i_proj"]["qkv_proj"]["weight"]
    o = att["o_proj"]["weight"]
    num_layers = o.shape[0]
    nkv = num_kv_heads or num_heads
    out = {"model.embed_tokens.weight": dec["emb"]["token_emb"]["weight"],
           "model.norm.weight": dec["output_norm"]["scale"]}
    for i in range(num_layers):
        if qkv.dim() == 5:                                             # [L, 3, D, N, H]
            q, k, v = qkv[i, 0], qkv[i, 1], qkv[i, 2]
        else:                                                          # [L, D, N + 2 Nkv, H]
            q, k, v = qkv[i][:, :num_heads], qkv[i][:, num_heads:num_heads + nkv], qkv[i][:, num_heads + nkv:]
        d = q.shape[0]
        pre = f"model.layers.{i}."
        out[pre + "self_attn.q_proj.weight"] = _pairs_to_halves(q).reshape(d, -1).t()
        out[pre + "self_attn.k_proj.weight"] = _pairs_to_halves(k).reshape(d, -1).t()
        out[pre + "self_attn.v_proj.weight"] = v.reshape(d, -1).t()
        out[pre + "self_attn.o_proj.weight"] = o[i].reshape(d, -1)
        out[pre + "input_layernorm.weight"] = layer["self_attention"]["norm"]["scale"][i]
        out[pre + "post_attention_layernorm.weight"] = layer["feed_forward"]["norm"]["scale"][i]
        out[pre + "mlp.gate_proj.weight"] = layer["feed_forward"]["linear1_0"]["weight"][i].t()
        out[pre + "mlp.up_proj.weight"] = layer["feed_forward"]["linear1_1"]["weight"][i].t()
        out[pre + "mlp.down_proj.weight"] = layer["feed_forward"]["linear2"]["weight"][i].t()
    head = dec.get("lm_head", {}).get("weight") if isinstance(dec.get("lm_head"), Mapping) else None
    out["lm_head.weight"] = head if head is not None else dec["emb"]["token_emb"]["weight"]
    return {k: v.contiguous() for k, v in out.items()}


def _contiguous(tree: Any) -> Any:
    if isinstance(tree, Mapping):
        return {k: _contiguous(v) for k, v in tree.items()}
    return tree.contiguous()


# ------------------------------------------------------------------------------------------
# T5 (the counterpart of the reference's T5X converter, axlearn/common/t5x_param_converter.py:
# checkpoints of the public T5 family reach this framework through their Hugging Face form).
# ------------------------------------------------------------------------------------------


def t5_hf_to_encoder_decoder(state_dict: Mapping[str, Tensor], *, num_heads: int, num_encoder_layers: int,
                             num_decoder_layers: int) -> dict:
    """``T5ForConditionalGeneration.state_dict()`` (gated feed-forward, i.e. v1.1 / UL2 style) -> the
    parameter tree of ``t5_encoder_decoder_config``.  T5 does not scale attention logits; this
    framework divides by ``sqrt(head_dim)``, so the query projections are multiplied by it."""
    sd = state_dict
    d = sd["shared.weight"].shape[1]
    inner = sd["encoder.block.0.layer.0.SelfAttention.q.weight"].shape[0]
    h = inner // num_heads

    def proj(w: Tensor, scale: float = 1.0) -> Tensor:       # [N*H, D] -> [D, N, H]
        return (w.t() * scale).reshape(d, num_heads, h).contiguous()

    def attention(prefix: str) -> dict:
        return {"i_proj": {"q_proj": {"weight": proj(sd[prefix + "q.weight"], h ** 0.5)},
                           "k_proj": {"weight": proj(sd[prefix + "k.weight"])},
                           "v_proj": {"weight": proj(sd[prefix + "v.weight"])}},
                "o_proj": {"weight": sd[prefix + "o.weight"].reshape(d, num_heads, h).contiguous()}}

    def ffn(prefix: str, norm: str) -> dict:
        return {"linear1_0": {"weight": sd[prefix + "wi_0.weight"].t().contiguous()},
                "linear1_1": {"weight": sd[prefix + "wi_1.weight"].t().contiguous()},
                "linear2": {"weight": sd[prefix + "wo.weight"].t().contiguous()},
                "norm": {"scale": sd[norm]}}

    enc_layers, dec_layers = {}, {}
    for i in range(num_encoder_layers):
        p = f"encoder.block.{i}.layer."
        enc_layers[f"layer{i}"] = {
            "self_attention": {"attention": attention(p + "0.SelfAttention."), "norm": {"scale": sd[p + "0.layer_norm.weight"]}},
            "feed_forward": ffn(p + "1.DenseReluDense.", p + "1.layer_norm.weight")}
    for i in range(num_decoder_layers):
        p = f"decoder.block.{i}.layer."
        dec_layers[f"layer{i}"] = {
            "self_attention": {"attention": attention(p + "0.SelfAttention."), "norm": {"scale": sd[p + "0.layer_norm.weight"]}},
            "cross_attention": {"attention": attention(p + "1.EncDecAttention."), "norm": {"scale": sd[p + "1.layer_norm.weight"]}},
            "feed_forward": ffn(p + "2.DenseReluDense.", p + "2.layer_norm.weight")}
    rel = "block.0.layer.0.SelfAttention.relative_attention_bias.weight"
    out = {
        "encoder": {"emb": {"token_emb": {"weight": sd["shared.weight"]}},
                    "relative_pos_emb": {"emb": {"weight": sd["encoder." + rel]}},
                    "transformer": enc_layers, "output": {"norm": {"scale": sd["encoder.final_layer_norm.weight"]}}},
        "decoder": {"emb": {"token_emb": {"weight": sd["shared.weight"]}},
                    "attention_mask": {"relative_pos_emb": {"emb": {"weight": sd["decoder." + rel]}}},
                    "transformer": dec_layers, "output_norm": {"scale": sd["decoder.final_layer_norm.weight"]}},
    }
    if "lm_head.weight" in sd:
        out["decoder"]["lm_head"] = {"weight": sd["lm_head.weight"]}
    return out
