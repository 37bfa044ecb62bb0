"""Micro-benchmarks of the sm_100a kernels against the measured roofline.

``python -m axlearn_b200.ops.kernel_bench --op gemm --m 16384 --n 4096 --k 4096`` times one
kernel with CUDA events (warm-up, L2 flushed between iterations by writing a 256 MiB buffer)
and prints one JSON line with the achieved TFLOP/s or GB/s, the fraction of the measured peak
(``MEASURED_PEAKS.json`` when present: cuBLAS bf16 burst throughput and copy bandwidth), and
the same measurement for the PyTorch library op for context.  The small default shapes are
also the ones used for ``ncu`` captures.

Ops: gemm (``--layout nn|nt|tn``: forward, data-gradient and weight-gradient operand forms),
gemm_fp8, grouped_gemm, decode_attn,
flash_fwd, flash_bwd, rmsnorm, swiglu, rope, ce, adamw.
"""

from __future__ import annotations

import argparse
import json
import math
import os

import torch

from axlearn_b200.ops import attention_ops, cuda_ops, flash_sm100


def _peaks() -> dict:
    here = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    path = os.path.join(here, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        return {"tflops": d["bf16_tflops"], "tflops_sustained": d.get("bf16_tflops_sustained"),
                "gbs": d["hbm_gbs"], "source": "measured"}
    return {"tflops": 1590.0, "tflops_sustained": 1400.0, "gbs": 6650.0, "source": "fallback"}


def _time(fn, iters: int, warmup: int = 3, flush: bool = True) -> float:
    """Median milliseconds per call."""
    scratch = torch.empty(256 << 20, dtype=torch.uint8, device="cuda") if flush else None
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    times = []
    for _ in range(iters):
        if scratch is not None:
            scratch.fill_(1)
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        fn()
        e.record()
        torch.cuda.synchronize()
        times.append(s.elapsed_time(e))
    times.sort()
    return times[len(times) // 2]


def bench_gemm(args) -> dict:
    m, n, k = args.m, args.n, args.k
    dev = "cuda"
    if args.layout == "nn":    # y = x @ w          (w stored [K, N])
        a = torch.randn(m, k, device=dev).bfloat16()
        b = torch.randn(k, n, device=dev).bfloat16()
    elif args.layout == "nt":  # dx = dy @ w^T      (w stored [N, K] row-major as seen here)
        a = torch.randn(m, k, device=dev).bfloat16()
        b = torch.randn(n, k, device=dev).bfloat16().t()
    else:                      # dw = x^T @ dy      (x stored [K, M])
        a = torch.randn(k, m, device=dev).bfloat16().t()
        b = torch.randn(k, n, device=dev).bfloat16()
    out = torch.empty(m, n, device=dev, dtype=torch.bfloat16)
    ours = _time(lambda: cuda_ops.gemm(a, b, out=out), args.iters)
    lib = _time(lambda: torch.matmul(a, b, out=out), args.iters)
    cuda_ops.check_status()
    flops = 2.0 * m * n * k
    return {"ms": ours, "tflops": flops / ours / 1e9, "library_ms": lib, "library_tflops": flops / lib / 1e9,
            "flops": flops}


def bench_gemm_fp8(args) -> dict:
    """Block-scaled fp8 GEMM (1x128 activation scales, 128x128 weight scales); the library
    column is the bf16 library GEMM of the same shape."""
    from axlearn_b200.ops import fp8_ops

    m, n, k = args.m, args.n, args.k
    a = torch.randn(m, k, device="cuda").bfloat16()
    b = torch.randn(n, k, device="cuda").bfloat16()
    aq, sa = fp8_ops.quantize_rows(a)
    bq, sb = fp8_ops.quantize_blocks(b)
    ours = _time(lambda: fp8_ops.gemm_fp8(aq, bq, sa, sb, a_gran=1), args.iters)
    out = torch.empty(m, n, device="cuda", dtype=torch.bfloat16)
    lib = _time(lambda: torch.matmul(a, b.t(), out=out), args.iters)
    quant = _time(lambda: fp8_ops.quantize_rows(a), args.iters)
    cuda_ops.check_status()
    flops = 2.0 * m * n * k
    return {"ms": ours, "tflops": flops / ours / 1e9, "library_ms": lib, "library_tflops": flops / lib / 1e9,
            "flops": flops, "quantize_rows_ms": quant, "quantize_rows_gbs": 3.0 * m * k / quant / 1e6}


def bench_grouped_gemm(args) -> dict:
    """Grouped GEMM of a drop-free MoE projection: ``--m`` (token, choice) pairs spread unevenly
    over ``--experts`` experts, ``[K, N]`` weights per expert; forward form and (``--layout tn``)
    the per-expert weight-gradient form.  The library column runs one matmul per expert over the
    same row ranges (offsets already on the host)."""
    from axlearn_b200.ops import moe_ops

    m, n, k, e = args.m, args.n, args.k, args.experts
    torch.manual_seed(0)
    probs = torch.softmax(torch.randn(e) * 0.5, 0)
    experts = torch.multinomial(probs, m, replacement=True).cuda()
    dest, offsets, block_expert, rows = moe_ops.padded_group_layout(experts, e)
    x = torch.zeros(rows, k, device="cuda", dtype=torch.bfloat16)
    x[dest.long()] = torch.randn(m, k, device="cuda").bfloat16()
    w = torch.randn(e, k, n, device="cuda").bfloat16()
    dy = torch.zeros(rows, n, device="cuda", dtype=torch.bfloat16)
    dy[dest.long()] = torch.randn(m, n, device="cuda").bfloat16()
    bounds = offsets.tolist()
    if args.layout == "tn":
        ours = _time(lambda: moe_ops._tgmm_kernel(x, dy, offsets, e), args.iters)  # pylint: disable=protected-access
        lib = _time(lambda: [x[bounds[i]:bounds[i + 1]].t() @ dy[bounds[i]:bounds[i + 1]] for i in range(e)], args.iters)
    else:
        ours = _time(lambda: moe_ops._gmm_kernel(x, w, block_expert, False), args.iters)  # pylint: disable=protected-access
        lib = _time(lambda: [x[bounds[i]:bounds[i + 1]] @ w[i] for i in range(e)], args.iters)
    cuda_ops.check_status()
    flops = 2.0 * bounds[-1] * n * k
    return {"ms": ours, "tflops": flops / ours / 1e9, "library_ms": lib, "library_tflops": flops / lib / 1e9,
            "flops": flops, "padded_rows": bounds[-1], "pairs": m}


def bench_flash(args, backward: bool) -> dict:
    b, t, n, nkv, h = args.batch, args.seq, args.heads, args.kv_heads or args.heads, args.head_dim
    q = torch.randn(b, t, n, h, device="cuda").bfloat16()
    k = torch.randn(b, t, nkv, h, device="cuda").bfloat16()
    v = torch.randn(b, t, nkv, h, device="cuda").bfloat16()
    scale = 1.0 / math.sqrt(h)
    causal = not args.full
    fwd_flops = 4.0 * b * n * t * t * h * (0.5 if causal else 1.0)
    if not backward:
        ours = _time(lambda: flash_sm100.forward(q, k, v, causal=causal, scale=scale), args.iters)
        qt, kt, vt = (x.transpose(1, 2) for x in (q, k, v))
        lib = _time(lambda: torch.nn.functional.scaled_dot_product_attention(
            qt, kt, vt, is_causal=causal, enable_gqa=nkv != n), args.iters)
        flops = fwd_flops
    else:
        out, lse = flash_sm100.forward(q, k, v, causal=causal, scale=scale)
        do = torch.randn_like(out)
        ours = _time(lambda: flash_sm100.backward(q, k, v, out, lse, do, causal=causal, scale=scale), args.iters)
        qt, kt, vt = (x.transpose(1, 2).detach().requires_grad_() for x in (q, k, v))
        o = torch.nn.functional.scaled_dot_product_attention(qt, kt, vt, is_causal=causal, enable_gqa=nkv != n)
        dot = do.transpose(1, 2)
        lib = _time(lambda: torch.autograd.grad(o, (qt, kt, vt), dot, retain_graph=True), args.iters)
        flops = 2.5 * fwd_flops  # 5 GEMMs in the minimal backward (this kernel pair issues 7)
    cuda_ops.check_status()
    return {"ms": ours, "tflops": flops / ours / 1e9, "library_ms": lib, "library_tflops": flops / lib / 1e9,
            "flops": flops}


def bench_decode_attn(args) -> dict:
    """Paged decode attention: ``--batch`` sequences of ``--seq`` cached tokens, ``--heads`` query /
    ``--kv_heads`` KV heads, 16-token pages; the library column is SDPA over the gathered dense cache."""
    from axlearn_b200.ops import decode_ops

    b, t, nq, nkv, h, ps = args.batch, args.seq, args.heads, args.kv_heads or args.heads, args.head_dim, 16
    pages = t // ps
    k = torch.randn(b * pages, ps, nkv, h, device="cuda").bfloat16()
    v = torch.randn(b * pages, ps, nkv, h, device="cuda").bfloat16()
    table = torch.randperm(b * pages, device="cuda").to(torch.int32).reshape(b, pages).contiguous()
    lengths = torch.full((b,), t, dtype=torch.int32, device="cuda")
    q = torch.randn(b, nq, h, device="cuda").bfloat16()
    splits = args.splits or decode_ops.default_splits(b, nkv, nq // nkv, t, ps)
    scratch = torch.empty(decode_ops._lib().axb_decode_attn_scratch_floats(b, nq, splits), device="cuda")  # pylint: disable=protected-access
    out = torch.empty_like(q)
    ours = _time(lambda: decode_ops.paged_decode_attention(q, k, v, table, lengths, splits=splits, out=out,
                                                           scratch=scratch), args.iters)
    kd = k.reshape(b, t, nkv, h).transpose(1, 2)
    vd = v.reshape(b, t, nkv, h).transpose(1, 2)
    qd = q[:, :, None, :]
    lib = _time(lambda: torch.nn.functional.scaled_dot_product_attention(qd, kd, vd, enable_gqa=nkv != nq), args.iters)
    cuda_ops.check_status()
    nbytes = 2 * k.numel() * 2
    return {"ms": ours, "gbs": nbytes / ours / 1e6, "library_ms": lib, "library_gbs": nbytes / lib / 1e6,
            "bytes": nbytes, "kv_splits": splits}


def bench_memory_bound(args) -> dict:
    rows, d = args.m, args.n
    x = torch.randn(rows, d, device="cuda").bfloat16()
    if args.op == "rmsnorm":
        scale = torch.ones(d, device="cuda").bfloat16()
        ours = _time(lambda: cuda_ops.rms_norm(x, scale, 1e-5), args.iters)
        lib = _time(lambda: torch.nn.functional.rms_norm(x, (d,), scale, 1e-5), args.iters)
        nbytes = 2 * x.numel() * 2
    elif args.op in ("rmsnorm_add", "rmsnorm_bwd", "rmsnorm_bwd_add"):
        # The fused forms of the training step: forward with the residual add (reads two rows,
        # writes the sum and the normalised row), backward without / with the residual branch's
        # gradient added in (reads x, dy [, dres], writes dx; dscale partials are small).
        scale = torch.ones(d, device="cuda").bfloat16()
        other = torch.randn_like(x)
        y, _, rstd = cuda_ops._rmsnorm_forward(x, None, scale, 1e-5)  # pylint: disable=protected-access
        if args.op == "rmsnorm_add":
            ours = _time(lambda: cuda_ops._rmsnorm_forward(x, other, scale, 1e-5), args.iters)  # pylint: disable=protected-access
            lib = _time(lambda: torch.nn.functional.rms_norm(x + other, (d,), scale, 1e-5), args.iters)
            nbytes = 4 * x.numel() * 2
        else:
            dres = other if args.op == "rmsnorm_bwd_add" else None
            ours = _time(lambda: cuda_ops._rmsnorm_backward(x, scale, rstd, y, dres), args.iters)  # pylint: disable=protected-access
            xg = x.clone().requires_grad_()

            def lib_fn():
                out = torch.nn.functional.rms_norm(xg, (d,), scale, 1e-5)
                (gx,) = torch.autograd.grad(out, xg, y)
                return gx if dres is None else gx + dres

            lib = _time(lib_fn, args.iters)
            nbytes = (4 if dres is not None else 3) * x.numel() * 2
    elif args.op == "swiglu":
        y = torch.randn_like(x)
        ours = _time(lambda: cuda_ops.swiglu(x, y), args.iters)
        lib = _time(lambda: torch.nn.functional.silu(x) * y, args.iters)
        nbytes = 3 * x.numel() * 2
    elif args.op == "rope":
        xr = x.reshape(1, rows, d // 128, 128)
        pos = torch.arange(rows, device="cuda")
        ours = _time(lambda: cuda_ops.rope(xr, pos, 1e4), args.iters)
        from axlearn_b200.ops import reference

        lib = _time(lambda: reference.rope(xr, pos, 1e4), args.iters)
        nbytes = 2 * x.numel() * 2
    elif args.op == "ce":
        tg = torch.randint(0, d, (rows,), device="cuda")
        live = torch.ones(rows, dtype=torch.bool, device="cuda")
        inv = torch.tensor(1.0 / rows, device="cuda")
        ours = _time(lambda: cuda_ops.ce_chunk(x, tg, live, 0.0, inv, True), args.iters)
        xf = x.clone().requires_grad_()
        lib = _time(lambda: torch.autograd.grad(torch.nn.functional.cross_entropy(xf.float(), tg), xf), args.iters)
        nbytes = 2 * x.numel() * 2
    else:  # adamw
        n = rows * d
        p, m, v = (torch.randn(n, device="cuda") for _ in range(3))
        v.abs_()
        g = torch.randn(n, device="cuda").bfloat16()
        sh = torch.empty(n, device="cuda", dtype=torch.bfloat16)
        ours = _time(lambda: cuda_ops.multi_tensor_adamw([p], [g], [m], [v], [sh], [1.0], step=2, lr=1e-3,
                                                         weight_decay=0.1, b1=0.9, b2=0.95, eps=1e-8), args.iters)
        opt = torch.optim.AdamW([p.requires_grad_()], lr=1e-3, fused=True)
        p.grad = g.float()
        lib = _time(opt.step, args.iters)
        nbytes = n * (4 + 2 + 4 + 4 + 4 + 4 + 4 + 2)
    return {"ms": ours, "gbs": nbytes / ours / 1e6, "library_ms": lib, "library_gbs": nbytes / lib / 1e6,
            "bytes": nbytes}


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--op", required=True,
                    choices=["gemm", "gemm_fp8", "grouped_gemm", "flash_fwd", "flash_bwd", "decode_attn", "rmsnorm", "rmsnorm_add", "rmsnorm_bwd", "rmsnorm_bwd_add", "swiglu", "rope", "ce",
                             "adamw"])
    ap.add_argument("--m", type=int, default=4096)
    ap.add_argument("--n", type=int, default=4096)
    ap.add_argument("--k", type=int, default=4096)
    ap.add_argument("--layout", default="nn", choices=["nn", "nt", "tn"])
    ap.add_argument("--experts", type=int, default=8)
    ap.add_argument("--batch", type=int, default=2)
    ap.add_argument("--seq", type=int, default=4096)
    ap.add_argument("--heads", type=int, default=32)
    ap.add_argument("--kv_heads", type=int, default=None)
    ap.add_argument("--head_dim", type=int, default=128)
    ap.add_argument("--full", action="store_true", help="non-causal attention")
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--splits", type=int, default=0, help="decode_attn: KV splits (0 = the default heuristic)")
    args = ap.parse_args()
    peaks = _peaks()
    if args.op == "gemm":
        r = bench_gemm(args)
    elif args.op == "gemm_fp8":
        r = bench_gemm_fp8(args)
    elif args.op == "grouped_gemm":
        r = bench_grouped_gemm(args)
    elif args.op == "decode_attn":
        r = bench_decode_attn(args)
    elif args.op in ("flash_fwd", "flash_bwd"):
        r = bench_flash(args, backward=args.op == "flash_bwd")
    else:
        r = bench_memory_bound(args)
    if "tflops" in r:
        r["frac_of_peak"] = r["tflops"] / peaks["tflops"]
        r["library_frac_of_peak"] = r["library_tflops"] / peaks["tflops"]
    else:
        r["frac_of_peak"] = r["gbs"] / peaks["gbs"]
        r["library_frac_of_peak"] = r["library_gbs"] / peaks["gbs"]
    r["peak_source"] = peaks["source"]
    r["op"] = args.op
    r["args"] = {k: v for k, v in vars(args).items() if k != "op"}
    print(json.dumps(r))


if __name__ == "__main__":
    main()
