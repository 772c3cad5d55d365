"""Where the time of one training step goes: kernel time shares of a Llama-3-8B-shaped model cut to a few
layers (full width, vocabulary and sequence length), from torch.profiler on one GPU.

    python benchmarks/step_breakdown.py --layers 4 --engine native

Prints the CUDA-event time of a step without the profiler first (the number to quote), then the table of
kernels sorted by device time (shares only: a profiler is attached for that step). With ``--no-profiler`` only
the timing runs, e.g. under ``ncu --metrics gpu__time_duration.sum`` for a launch list.
"""

from __future__ import annotations

import argparse
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch  # noqa: E402
import torch.distributed as dist  # noqa: E402
from torch.profiler import ProfilerActivity, profile  # noqa: E402

import moodist_b200  # noqa: E402,F401
from moodist_b200.models.llama import LlamaConfig  # noqa: E402
from moodist_b200.parallel.fsdp import ShardedTrainer  # noqa: E402
from moodist_b200.utils.testing import free_port  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--layers", type=int, default=4)
    ap.add_argument("--engine", default="native", choices=["native", "fsdp2"])
    ap.add_argument("--rows", type=int, default=40)
    ap.add_argument("--no-profiler", action="store_true",
                    help="only time the steps (for runs under an external profiler such as ncu's launch list)")
    args = ap.parse_args()
    torch.cuda.set_device(0)
    dist.init_process_group("moodist", init_method=f"tcp://127.0.0.1:{free_port()}", rank=0, world_size=1)
    cfg = LlamaConfig.llama3_8b()
    cfg.n_layers = args.layers
    tr = ShardedTrainer(cfg, engine=args.engine)
    toks = [torch.randint(0, cfg.vocab_size, (1, cfg.max_seq_len + 1), device="cuda") for _ in range(6)]
    for i in range(3):
        tr.step_on_device(toks[i])
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    tr.step_on_device(toks[3])
    tr.step_on_device(toks[4])
    e1.record()
    torch.cuda.synchronize()
    print(f"{args.layers} layers, engine {args.engine}: {e0.elapsed_time(e1) / 2:.2f} ms/step (CUDA events, no profiler)")
    if args.no_profiler:
        dist.destroy_process_group()
        return
    with profile(activities=[ProfilerActivity.CUDA, ProfilerActivity.CPU]) as prof:
        tr.step_on_device(toks[5])
        torch.cuda.synchronize()
    print(prof.key_averages().table(sort_by="self_cuda_time_total", row_limit=args.rows, max_name_column_width=70))
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
