"""Where one training step of the Llama-3-8B-shaped model spends its time, per CUDA stream.

    python benchmarks/step_timeline.py regather one_gpu
    torchrun --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 benchmarks/step_timeline.py regather two_gpus
    torchrun ... benchmarks/step_timeline.py resident two_gpus_resident
    torchrun ... benchmarks/step_timeline.py regather two_gpus_unfused fused=0

Runs a few steps of `ShardedTrainer`, times two of them with CUDA events (no profiler attached), then records
ONE more step with torch.profiler (CUPTI kernel activity) and writes, for rank 0, `step_timeline_<tag>.json`:
per stream the number of kernels, their summed time, the idle time between them, the largest gaps and the
kernels that account for most of the time; plus how much GEMM time overlapped work of another stream. Times
taken under the profiler are for shares and ordering only; the step time to quote is `plain_ms_per_step`.
The reference has no trainer; this is a diagnostic for the engines in `moodist_b200/parallel`."""
import os, sys, json, collections, torch, torch.distributed as dist
sys.path.insert(0, os.getcwd())
import moodist_b200
from moodist_b200.models.llama import LlamaConfig
from moodist_b200.parallel.fsdp import ShardedTrainer
from torch.profiler import profile, ProfilerActivity

rank = int(os.environ.get("RANK", "0")); world = int(os.environ.get("WORLD_SIZE", "1"))
os.environ.setdefault("MASTER_ADDR", "127.0.0.1"); os.environ.setdefault("MASTER_PORT", "29544")
torch.cuda.set_device(rank)
dist.init_process_group("moodist", rank=rank, world_size=world)
schedule, tag = sys.argv[1], sys.argv[2]
kw = {}
for a in sys.argv[3:]:
    k, v = a.split("="); kw[k] = (v == "1")
cfg = LlamaConfig.llama3_8b()
tr = ShardedTrainer(cfg, schedule=schedule, **kw)
toks = [torch.randint(0, cfg.vocab_size, (1, 8193), device="cuda") for _ in range(6)]
for i in range(3): tr.step_on_device(toks[i])
tr.engine.wait(); torch.cuda.synchronize(); dist.barrier()
e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
e0.record(); tr.step_on_device(toks[3]); tr.step_on_device(toks[4]); tr.engine.wait(); e1.record(); torch.cuda.synchronize()
plain_ms = e0.elapsed_time(e1) / 2
dist.barrier()
with profile(activities=[ProfilerActivity.CUDA]) as prof:
    tr.step_on_device(toks[5]); tr.engine.wait(); torch.cuda.synchronize()
if rank == 0:
    path = f"/tmp/trace_{tag}.json"
    prof.export_chrome_trace(path)
    ev = [e for e in json.load(open(path))["traceEvents"] if e.get("cat") in ("kernel", "gpu_memcpy", "gpu_memset") and "dur" in e]
    by_stream = collections.defaultdict(list)
    for e in ev: by_stream[e["args"].get("stream")].append(e)
    t0 = min(e["ts"] for e in ev); t1 = max(e["ts"] + e["dur"] for e in ev)
    def short(n):
        n = n.replace("void ", "")
        for pre in ("mb::gemm::", "mb::coll::", "mb::fused::", "at::native::", "(anonymous namespace)::"):
            n = n.replace(pre, "")
        return n[:70]
    out = {"tag": tag, "plain_ms_per_step": plain_ms, "profiled_span_ms": (t1 - t0) / 1e3, "streams": {}}
    main = max(by_stream, key=lambda s: sum(e["dur"] for e in by_stream[s]))
    for s, lst in by_stream.items():
        lst.sort(key=lambda e: e["ts"])
        busy = 0.0; cur_end = None; gaps = []
        for e in lst:
            if cur_end is None: cur_end = e["ts"]
            if e["ts"] > cur_end:
                gaps.append((e["ts"] - cur_end, short(e["name"])))
                busy += 0
            cur_end = max(cur_end, e["ts"] + e["dur"])
        names = collections.Counter(); cnt = collections.Counter()
        for e in lst: names[short(e["name"])] += e["dur"]; cnt[short(e["name"])] += 1
        tot = sum(e["dur"] for e in lst)
        gaps.sort(reverse=True)
        out["streams"][str(s) + (" (main)" if s == main else "")] = {
            "kernels": len(lst), "sum_ms": tot / 1e3, "idle_ms": sum(g for g, _ in gaps) / 1e3,
            "top_gaps_us": [(round(g), n) for g, n in gaps[:12]],
            "top": [(n, round(d / 1e3, 2), cnt[n]) for n, d in names.most_common(14)]}
    # GEMM kernels on the main stream: time while some other stream is busy vs not
    others = sorted((e["ts"], e["ts"] + e["dur"]) for s, l in by_stream.items() if s != main for e in l)
    def overlap(a, b):
        tot = 0.0
        for x, y in others:
            if y <= a: continue
            if x >= b: break
            tot += min(b, y) - max(a, x)
        return tot
    g_over = g_alone = 0.0; stats = collections.defaultdict(lambda: [0, 0.0, 0, 0.0])
    for e in by_stream[main]:
        if "gemm" not in e["name"]: continue
        a, b = e["ts"], e["ts"] + e["dur"]
        frac = overlap(a, b) / max(e["dur"], 1e-9)
        key = (short(e["name"])[:40], e["args"].get("grid"), round(e["dur"] / 50))
        if frac > 0.5: g_over += e["dur"]
        else: g_alone += e["dur"]
    out["gemm_ms_overlapped_with_side_stream"] = g_over / 1e3
    out["gemm_ms_alone"] = g_alone / 1e3
    json.dump(out, open(f"step_timeline_{tag}.json", "w"), indent=1)
    print(json.dumps(out)[:3000])
dist.barrier()
dist.destroy_process_group()
