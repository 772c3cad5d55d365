"""Sharded training of a Llama-shaped decoder on the GPUs of one machine.

    python examples/train_llama_sharded.py --model tiny --steps 20                       # one GPU
    torchrun --nproc-per-node 8 examples/train_llama_sharded.py --model llama3-8b --steps 10

Every rank trains on its own random token batches (synthetic data).  By default the FSDP2 schedule runs
(``moodist_b200.parallel.regather.RegatherEngine``: weights sharded by rows at rest, gathered per block, the QKV
and gate/up gathers fused into their GEMMs); ``--schedule resident`` keeps gathered parameters on every GPU
(``moodist_b200.parallel.sharded.ShardedEngine``).  Both run over the "moodist" backend.
"""

import argparse
import os
import sys
import time

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import moodist_b200  # noqa: E402,F401  (registers the backend)
from moodist_b200.models.llama import LlamaConfig  # noqa: E402
from moodist_b200.parallel.fsdp import ShardedTrainer  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="tiny", choices=["tiny", "llama3-8b"])
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--seq-len", type=int, default=0, help="0: the model's maximum")
    ap.add_argument("--lr", type=float, default=3e-4)
    ap.add_argument("--schedule", default="regather", choices=["regather", "resident"])
    ap.add_argument("--checkpoint", default="", help="directory for one shard file per rank at the end")
    args = ap.parse_args()

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29555")
    torch.cuda.set_device(local)
    dist.init_process_group("moodist", rank=rank, world_size=world)

    cfg = LlamaConfig.llama3_8b() if args.model == "llama3-8b" else LlamaConfig.tiny()
    seq = args.seq_len or cfg.max_seq_len
    trainer = ShardedTrainer(cfg, lr=args.lr, schedule=args.schedule)
    gen = torch.Generator().manual_seed(rank)
    t0 = time.time()
    for step in range(args.steps):
        tokens = torch.randint(0, cfg.vocab_size, (1, seq + 1), generator=gen).pin_memory()
        loss = trainer.step(tokens)  # H2D copy, forward, backward, sharded optimizer step
        if rank == 0 and (step % 5 == 0 or step + 1 == args.steps):
            print(f"step {step:4d}  loss {loss:.4f}  {(time.time() - t0) / (step + 1) * 1e3:.0f} ms/step")
    if args.checkpoint:
        os.makedirs(args.checkpoint, exist_ok=True)
        torch.save(trainer.engine.state_dict(), os.path.join(args.checkpoint, f"shard-{rank:03d}-of-{world:03d}.pt"))
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
