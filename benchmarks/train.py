#!/usr/bin/env python
"""Async data-parallel training on a shared tensor vs. synchronous all-reduce training.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port 29500 \
        benchmarks/train.py --model char_rnn|gpt2 --mode async|sync --steps 200 [--out train.json]

char_rnn: 2-layer LSTM, hidden 512, vocabulary 65, sequence 50, batch 64 per GPU, fp32, SGD lr 2e-3, all
          parameters in one shared tensor.
gpt2:     GPT-2 small, sequence 1024, micro-batch 8 per GPU, bf16 compute over fp32 master weights held in a shared
          arena (table layout: every parameter tensor starts on a scale-block boundary).
Data: synthetic uniform-random token ids (there is nothing to learn beyond the unigram entropy; the runs compare
loss-versus-wall-clock curves and throughput).  Rank 0 prints one JSON line: tokens/s over all ranks, exposed
synchronisation time (fraction of the step the training stream spends in pull/push), loss samples.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
from pathlib import Path

sys.path.insert(0, str(Path(__file__).resolve().parent.parent))

import torch  # noqa: E402
import torch.distributed as dist  # noqa: E402

import sharedtensor  # noqa: E402
from sharedtensor_b200.models import GPT2, CharRNN, GPT2Config, flatten_parameters  # noqa: E402
from sharedtensor_b200.parallel.trainers import (AsyncTrainer, SyncTrainer, random_token_batches,  # noqa: E402
                                                 structured_token_batches)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="char_rnn", choices=["char_rnn", "gpt2", "gpt2_tiny"])
    ap.add_argument("--mode", default="async", choices=["async", "sync"])
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--lr", type=float, default=None)
    ap.add_argument("--data", default="random", choices=["random", "structured"],
                    help="random: uniform tokens (the benchmark configs); structured: a learnable arithmetic sequence")
    ap.add_argument("--comm-ctas", type=int, default=148, help="SMs the sync rounds may use (async mode)")
    ap.add_argument("--round-interval-us", type=int, default=0,
                    help="engine-thread mode (--rounds-per-step 0): pause after every busy sync round")
    ap.add_argument("--rel-bits", type=int, default=14,
                    help="async mode: a block stops sending once its residual is below 2^-rel_bits of its largest value")
    ap.add_argument("--topology", default="tree", choices=["tree", "mesh"])
    ap.add_argument("--rounds-per-step", type=int, default=1,
                    help="async mode: > 0 = no engine thread, the trainer queues this many sync rounds behind every update; "
                         "0 = free-running engine thread")
    ap.add_argument("--out", default="")
    args = ap.parse_args()
    rank, local, world = int(os.environ.get("RANK", 0)), int(os.environ.get("LOCAL_RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29500")
    dist.init_process_group("gloo", rank=rank, world_size=world)
    nccl = dist.new_group(backend="nccl") if (world > 1 and args.mode == "sync") else None
    torch.manual_seed(0)  # every rank builds the same initial model
    if args.model == "char_rnn":
        model = CharRNN().to(dev)
        vocab, batch, seq, dtype, lr = 65, 64, 50, torch.float32, 2e-3
    else:
        cfg = GPT2Config() if args.model == "gpt2" else GPT2Config.tiny()
        model = GPT2(cfg).to(dev)
        vocab, batch, seq, dtype, lr = cfg.vocab, 8, cfg.ctx, torch.bfloat16, 1e-3
    if args.lr is not None:
        lr = args.lr
    make = random_token_batches if args.data == "random" else structured_token_batches
    batches = make(vocab, batch, seq, dev, seed=1000 + rank)
    shared = None
    if args.mode == "async":
        # fp32 masters, one arena; parameters start on scale-block boundaries (table layout)
        probe, _ = flatten_parameters(model, align=32, dtype=torch.float32)
        port = int(os.environ.get("MASTER_PORT", "29500")) + 31
        topo = {"topology": "mesh", "group_rank": rank, "group_size": world} if args.topology == "mesh" else {}
        for r in range(world):
            if r == rank or args.topology == "mesh":
                if shared is not None:
                    continue
                shared = sharedtensor.createOrFetch("127.0.0.1", port, probe if rank == 0 else torch.empty_like(probe),
                                                     comm_ctas=args.comm_ctas, round_interval_us=args.round_interval_us,
                                                     rel_bits=args.rel_bits, **topo,
                                                     **({"engine": "manual"} if args.rounds_per_step > 0 else {}))
            torch.cuda.synchronize()
            if args.topology == "tree":
                dist.barrier()
        trainer = AsyncTrainer(model, shared, lr=lr, param_dtype=dtype, rounds_per_step=args.rounds_per_step)
        del probe
    else:
        trainer = SyncTrainer(model, lr=lr, param_dtype=dtype, group=nccl)
    trainer.run(batches, steps=args.warmup, log_every=1000)
    trainer.log = type(trainer.log)()
    torch.cuda.synchronize()
    dist.barrier()
    log = trainer.run(batches, steps=args.steps, log_every=max(1, args.steps // 20))
    summ = log.summary()
    t = torch.tensor([summ["tokens_per_s"], summ["exposed_sync_frac"], summ["seconds"]], dtype=torch.float64)
    tot = t.clone()
    dist.all_reduce(tot, op=dist.ReduceOp.SUM)
    mx = t.clone()
    dist.all_reduce(mx, op=dist.ReduceOp.MAX)
    stats = shared.stats()["device"] if shared is not None else None
    torch.cuda.synchronize()
    dist.barrier()
    if shared is not None:
        shared.close()
    if rank == 0:
        out = {"model": args.model, "mode": args.mode, "n_gpus": world, "steps": args.steps,
               "tokens_per_s": float(tot[0]), "tokens_per_s_per_gpu": float(tot[0]) / world,
               "exposed_sync_frac_max": float(mx[1]), "seconds_max": float(mx[2]), "lr": lr, "dtype": str(dtype).replace("torch.", ""),
               "loss_curve": [[round(w, 4), round(l, 5)] for w, l in zip(log.wall, log.loss)], "device_status": stats, "rel_bits": args.rel_bits, "topology": args.topology,
               "comm_ctas": args.comm_ctas, "round_interval_us": args.round_interval_us,
               "rounds_per_step": args.rounds_per_step,
               "data": "synthetic uniform-random tokens" if args.data == "random" else "synthetic arithmetic token sequences", "parameters": trainer.flat.numel()}
        print(json.dumps(out), flush=True)
        if args.out:
            Path(args.out).write_text(json.dumps(out, indent=1))
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
