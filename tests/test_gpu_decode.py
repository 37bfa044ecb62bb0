"""Decode kernels and the decode engine against fp32 torch references (one GPU)."""

import math

import pytest
import torch

pytestmark = pytest.mark.gpu


def _pools(b, max_pages, page_size, nkv, h, seed=0):
    g = torch.Generator(device="cuda").manual_seed(seed)
    n_pages = b * max_pages + 3
    k = torch.randn(n_pages, page_size, nkv, h, device="cuda", generator=g).bfloat16()
    v = torch.randn(n_pages, page_size, nkv, h, device="cuda", generator=g).bfloat16()
    # A scrambled page table: sequences own arbitrary pages.
    perm = torch.randperm(n_pages, device="cuda", generator=g)[:b * max_pages].to(torch.int32)
    return k, v, perm.reshape(b, max_pages).contiguous()


@pytest.mark.parametrize("nq,nkv", [(4, 4), (8, 2), (8, 1), (6, 3), (8, 4), (16, 4), (32, 8)])
@pytest.mark.parametrize("splits", [1, 3])
def test_paged_decode_attention_matches_reference(nq, nkv, splits):
    from axlearn_b200.ops import cuda_ops, decode_ops

    b, page_size, max_pages, h = 5, 16, 9, 128
    k, v, table = _pools(b, max_pages, page_size, nkv, h)
    lengths = torch.tensor([1, 16, 17, 100, 144], dtype=torch.int32, device="cuda")
    q = torch.randn(b, nq, h, device="cuda").bfloat16()
    out = decode_ops.paged_decode_attention(q, k, v, table, lengths, splits=splits)
    ref = decode_ops.reference_paged_attention(q, k, v, table, lengths)
    torch.cuda.synchronize()
    cuda_ops.check_status()
    err = (out.float() - ref).abs().max().item()
    assert err < 2e-2 * max(1.0, ref.abs().max().item()), err


def test_rope_append_writes_page_slot_and_rotates():
    from axlearn_b200.ops import decode_ops, reference

    b, nq, nkv, h, page_size, max_pages = 3, 4, 2, 128, 16, 4
    k, v, table = _pools(b, max_pages, page_size, nkv, h, seed=1)
    k0, v0 = k.clone(), v.clone()
    lengths = torch.tensor([1, 16, 40], dtype=torch.int32, device="cuda")
    qkv = torch.randn(b, (nq + 2 * nkv) * h, device="cuda").bfloat16()
    q = decode_ops.rope_append_paged(qkv, k, v, table, lengths, num_q_heads=nq, theta=5e5)
    x = qkv.reshape(b, 1, nq + 2 * nkv, h)
    for i in range(b):
        pos = torch.tensor([int(lengths[i]) - 1], device="cuda")
        ref_q = reference.rope(x[i:i + 1, :, :nq].float(), pos, 5e5)[0, 0]
        ref_k = reference.rope(x[i:i + 1, :, nq:nq + nkv].float(), pos, 5e5)[0, 0]
        assert (q[i].float() - ref_q).abs().max() < 3e-2
        page = int(table[i, (int(lengths[i]) - 1) // page_size])
        off = (int(lengths[i]) - 1) % page_size
        assert (k[page, off].float() - ref_k).abs().max() < 3e-2
        assert torch.equal(v[page, off], x[i, 0, nq + nkv:])
        k0[page, off], v0[page, off] = k[page, off], v[page, off]
    # Nothing else was touched.
    assert torch.equal(k, k0) and torch.equal(v, v0)


def test_swiglu_packed():
    from axlearn_b200.ops import decode_ops

    gu = torch.randn(7, 2 * 96, device="cuda").bfloat16()
    out = decode_ops.swiglu_packed(gu)
    ref = torch.nn.functional.silu(gu[:, :96].float()) * gu[:, 96:].float()
    assert (out.float() - ref).abs().max() < 3e-2


def test_one_shot_all_reduce_emulated():
    """Four emulated ranks on one GPU: every rank pushes first (separate launches), then every
    rank finishes -- no launch waits on a later one."""
    from axlearn_b200.ops import cuda_ops, decode_ops

    world, n, sites = 4, 4096, 2
    ranks = [decode_ops.OneShotAllReduce(n, sites, device="cuda", peers=[None] * world, rank=r) for r in range(world)]
    for r in ranks:
        r.connect(ranks)
    for step in range(2):
        xs = [torch.randn(n, device="cuda").bfloat16() for _ in range(world)]
        res = torch.randn(n, device="cuda").bfloat16()
        for r in ranks:
            r.begin_step()
        for site in range(sites):
            for r, x in zip(ranks, xs):
                r.push(x, site)
            for r in ranks:
                out = r.finish(site, residual=res)
                ref = res.float() + sum(x.float() for x in xs)
                assert (out.float() - ref).abs().max() < 5e-2, (step, site)
    torch.cuda.synchronize()
    cuda_ops.check_status()


@pytest.mark.parametrize("world,m,k,n", [(2, 64, 256, 512), (2, 4096, 512, 1024), (4, 2048, 256, 2048)])
def test_gemm_with_all_reduce_push_epilogue_emulated(world, m, k, n):
    """Emulated ranks: each rank's GEMM stores its rows into every staging buffer and raises the
    flags itself; the finish kernels then see residual + the sum of the products.  The small case
    runs on the single-CTA kernel, the large ones on the CTA-pair kernel (TMA stores per peer)."""
    from axlearn_b200.ops import cuda_ops, decode_ops

    ranks = [decode_ops.OneShotAllReduce(m * n, 2, device="cuda", peers=[None] * world, rank=r) for r in range(world)]
    for r in ranks:
        r.connect(ranks)
    a = [torch.randn(m, k, device="cuda").bfloat16() for _ in range(world)]
    b = [(torch.randn(k, n, device="cuda") * 0.1).bfloat16() for _ in range(world)]
    res = torch.randn(m * n, device="cuda").bfloat16()
    for step in range(2):
        for r in ranks:
            r.begin_step()
        for r in range(world):
            ranks[r].gemm_push(a[r], b[r], 0)
        ref = res.float() + sum((x.float() @ y.float()).reshape(-1) for x, y in zip(a, b))
        for r in ranks:
            out = r.finish(0, residual=res)
            assert (out.float() - ref).abs().max() < 3e-2 * ref.abs().max(), step
    torch.cuda.synchronize()
    cuda_ops.check_status()


def _tiny_model(num_kv_heads):
    from axlearn_b200.common import prng
    from axlearn_b200.experiments.text.gpt import fuji

    cfg = fuji.model_config(num_layers=2, hidden_dim=256, num_heads=2, num_kv_heads=num_kv_heads, vocab_size=512,
                            rope_theta=1e4, shared_lm_head=False, ffn_dim=512)
    model = cfg.set(name="model").instantiate(parent=None)
    params = model.initialize_parameters_recursively(prng.PRNGKey(0))
    return model, params


@pytest.mark.parametrize("num_kv_heads,use_graph", [(None, True), (1, False)])
def test_decode_engine_matches_model_forward(num_kv_heads, use_graph):
    from axlearn_b200.common import prng
    from axlearn_b200.common.module import functional
    from axlearn_b200.inference.decode_engine import DecodeEngine, FujiDims, weights_from_fuji_state
    from axlearn_b200.ops import cuda_ops

    model, params = _tiny_model(num_kv_heads)
    dims = FujiDims(num_layers=2, hidden_dim=256, num_heads=2, num_kv_heads=num_kv_heads or 2, head_dim=128,
                    ffn_dim=512, vocab_size=512, rope_theta=1e4)
    weights = weights_from_fuji_state(params, dims, device="cuda")
    batch, t, new = 3, 128, 12
    engine = DecodeEngine(weights, dims, batch=batch, max_len=t + new + 4, device=torch.device("cuda"),
                          use_graph=use_graph)
    g = torch.Generator().manual_seed(0)
    prompts = torch.randint(2, 512, (batch, t), generator=g)
    tokens = engine.generate(prompts.cuda(), new).cpu()
    torch.cuda.synchronize()
    cuda_ops.check_status()
    assert engine.launches_per_step > 0
    # Teacher-forced fp32 logits of the reference model over prompt + generated tokens.
    from axlearn_b200.common.utils import tree_leaves

    full = torch.cat([prompts, tokens], dim=1).to(tree_leaves(params)[0].device)
    logits, _ = functional(model, prng.PRNGKey(1), params, dict(input_batch={"input_ids": full}),
                           is_training=False, method="extract_logits")
    for b in range(batch):
        for i in range(new):
            row = logits[b, t + i - 1].float().cpu()
            # The engine's pick is the reference argmax up to bf16 noise between near-ties.
            assert row.max() - row[tokens[b, i]] < 0.1 * max(1.0, row.std().item()), (b, i)


def test_sample_decode_api_runs_on_the_engine_and_matches_the_eager_path(monkeypatch):
    """``Model.sample_decode`` on a Fuji-shaped bf16 model on one GPU goes through the CUDA-graph
    engine; with deterministic sampling (top-k = 1) its tokens are those of the eager
    ``prefill_states`` / ``extend_step`` path, ragged prompts and two decodes per prompt included."""
    from axlearn_b200.common import decoding, logit_modifiers, prng
    from axlearn_b200.common.module import functional
    from axlearn_b200.common.utils import tree_map
    from axlearn_b200.inference import decode_engine
    from axlearn_b200.ops import cuda_ops

    model, params = _tiny_model(1)
    params = tree_map(lambda t: t.cuda().bfloat16() if t.is_floating_point() else t.cuda(), params)
    g = torch.Generator().manual_seed(3)
    prefix = torch.randint(2, 512, (3, 24), generator=g)
    prefix[1, 17:] = 0            # shorter prompts are right-padded with the pad id
    prefix[2, 9:] = 0
    calls = {"n": 0}
    real = decode_engine.DecodeEngine.step_logits

    def counted(self, tokens):
        calls["n"] += 1
        return real(self, tokens)

    monkeypatch.setattr(decode_engine.DecodeEngine, "step_logits", counted)
    kwargs = dict(input_batch={"prefix": prefix.cuda()}, num_decodes=2, max_sequence_length=40,
                  logits_modifier=logit_modifiers.top_k_logits(1),
                  stop_decoding_condition=decoding.StopOnSubsequence([[511]]))
    fast, _ = functional(model, prng.PRNGKey(5), params, kwargs, is_training=False, method="sample_decode")
    assert calls["n"] > 0, "the engine was not used"
    torch.cuda.synchronize()
    cuda_ops.check_status()
    monkeypatch.setenv("AXB200_DECODE_ENGINE", "0")
    before = calls["n"]
    slow, _ = functional(model, prng.PRNGKey(5), params, kwargs, is_training=False, method="sample_decode")
    assert calls["n"] == before
    assert fast.sequences.shape == slow.sequences.shape == (3, 2, 39)
    assert torch.equal(fast.sequences[:, :, :8], slow.sequences[:, :, :8])          # the prompts
    # With top-k = 1 every generated token must be the argmax of the model's own logits for the
    # sequence so far, up to bf16 noise between near-ties (a random model has many of those, so
    # the two paths may part ways at a tie and are therefore not compared token by token).
    lengths = (prefix != 0).sum(-1)
    for out in (fast, slow):
        full = torch.cat([prefix[:, :1].cuda().repeat_interleave(2, dim=0), out.sequences.reshape(6, 39)], dim=1)
        logits, _ = functional(model, prng.PRNGKey(1), params, dict(input_batch={"input_ids": full}),
                               is_training=False, method="extract_logits")
        for row in range(6):
            start = int(lengths[row // 2])
            for t in range(start, 40):
                tok = int(full[row, t])
                if tok == 0:
                    break
                ref = logits[row, t - 1].float()
                assert ref.max() - ref[tok] < 0.15 * max(1.0, ref.std().item()), (row, t)
    same = (fast.sequences == slow.sequences).float().mean().item()
    assert same > 0.5, same
