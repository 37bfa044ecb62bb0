"""Decode benchmark: prefill TTFT and per-token decode latency of a Fuji decoder.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \
        -m axlearn_b200.inference.bench_decode --model 7B --batch 64 --prompt-len 2048 --new-tokens 256

Tensor parallel over all ranks (``model`` = world size), random-init bf16 weights, uniform-random
prompt tokens from seed 0, greedy decoding, paged bf16 KV cache with 16-token pages.  Times are
CUDA-event times on each rank, reported as the max over ranks.  Prints one JSON line on rank 0.
"""

from __future__ import annotations

import argparse
import json
import os

import torch
import torch.distributed as dist

from axlearn_b200.inference.decode_engine import DecodeEngine, FujiDims, LayerWeights

MODELS = {
    "7B": FujiDims(num_layers=32, hidden_dim=4096, num_heads=32, num_kv_heads=32, head_dim=128, ffn_dim=11008,
                   vocab_size=32768, rope_theta=1e4),
    "1B": FujiDims(num_layers=16, hidden_dim=2048, num_heads=16, num_kv_heads=16, head_dim=128, ffn_dim=8192,
                   vocab_size=32768, rope_theta=1e4),
    "test": FujiDims(num_layers=2, hidden_dim=512, num_heads=8, num_kv_heads=8, head_dim=128, ffn_dim=1024,
                     vocab_size=2048, rope_theta=1e4),
}


def random_weights(dims: FujiDims, *, rank: int, world: int, device) -> dict:
    """Random-init weights of the architecture, created directly as this rank's shards.
    Replicated tensors use a rank-independent seed."""
    d, h = dims.hidden_dim, dims.head_dim
    nl, nkvl, fl = dims.num_heads // world, dims.num_kv_heads // world, dims.ffn_dim // world
    shared = torch.Generator(device=device).manual_seed(1234)
    local = torch.Generator(device=device).manual_seed(100 + rank)

    def rnd(gen, *shape, std):
        return (torch.randn(*shape, device=device, generator=gen, dtype=torch.float32) * std).to(torch.bfloat16)

    layers = []
    for _ in range(dims.num_layers):
        layers.append(LayerWeights(
            attn_norm=torch.ones(d, dtype=torch.bfloat16, device=device),
            wqkv=rnd(local, d, (nl + 2 * nkvl) * h, std=d ** -0.5),
            wo=rnd(local, nl * h, d, std=(dims.num_heads * h) ** -0.5),
            ffn_norm=torch.ones(d, dtype=torch.bfloat16, device=device),
            wgu=rnd(local, d, 2 * fl, std=d ** -0.5),
            wdown=rnd(local, fl, d, std=dims.ffn_dim ** -0.5)))
    return {
        "layers": layers,
        "emb": rnd(shared, dims.vocab_size, d, std=1.0),
        "head": rnd(shared, dims.vocab_size, d, std=d ** -0.5),
        "final_norm": torch.ones(d, dtype=torch.bfloat16, device=device),
    }


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="7B", choices=sorted(MODELS))
    ap.add_argument("--batch", type=int, default=64)
    ap.add_argument("--prompt-len", type=int, default=2048)
    ap.add_argument("--new-tokens", type=int, default=256)
    ap.add_argument("--page-size", type=int, default=16)
    ap.add_argument("--no-graph", action="store_true")
    args = ap.parse_args()

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    group = None
    if world > 1:
        dist.init_process_group("nccl", device_id=device)
        group = dist.group.WORLD
    dims = MODELS[args.model]
    weights = random_weights(dims, rank=rank, world=world, device=device)
    engine = DecodeEngine(weights, dims, batch=args.batch, max_len=args.prompt_len + args.new_tokens + 16,
                          page_size=args.page_size, group=group, device=device, use_graph=not args.no_graph)
    g = torch.Generator().manual_seed(0)
    prompts = torch.randint(0, dims.vocab_size, (args.batch, args.prompt_len), generator=g).to(device)

    def sync():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # Warm-up: one short prefill + a few steps (graph capture included), then the timed run
    # from a clean cache.
    engine.prefill(prompts)
    engine.decode(4)
    sync()
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(3)]
    ev[0].record()
    first = engine.prefill(prompts)
    ev[1].record()
    rest = engine.decode(args.new_tokens - 1)
    ev[2].record()
    sync()
    from axlearn_b200.ops import cuda_ops

    cuda_ops.check_status()
    t = torch.tensor([ev[0].elapsed_time(ev[1]), ev[1].elapsed_time(ev[2])], device=device)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ttft_ms, decode_ms = t.tolist()
    tokens = torch.cat([first[:, None], rest], dim=1)
    if world > 1:
        ref = tokens.clone()
        dist.broadcast(ref, src=0)
        same = bool((ref == tokens).all())
    else:
        same = True
    if rank == 0:
        steps = args.new_tokens - 1
        print(json.dumps({
            "metric": "Fuji decode: prefill TTFT and per-token latency (max over ranks)",
            "model": args.model, "n_gpus": world, "parallelism": f"model{world}", "batch": args.batch,
            "prompt_len": args.prompt_len, "new_tokens": args.new_tokens, "page_size": args.page_size,
            "ttft_ms": ttft_ms, "prefill_tokens_per_s": args.batch * args.prompt_len / (ttft_ms / 1e3),
            "decode_ms_per_token": decode_ms / steps, "decode_tokens_per_s": args.batch * steps / (decode_ms / 1e3),
            "kv_splits": engine.splits, "kernel_launches_per_step": engine.launches_per_step,
            "cuda_graph": not args.no_graph, "ranks_agree": same, "dtype": "bf16", "data": "synthetic",
        }))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
