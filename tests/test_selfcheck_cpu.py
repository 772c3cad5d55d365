"""The benchmark's correctness check (every collective against values each rank recomputes on the CPU) run on CPU
ranks over the host path: the oracle code is exercised without a GPU, and a wrong result is reported."""

import torch

from moodist_b200.utils.testing import init_moodist, run_ranks


def _body(rank, world, port):
    dist = init_moodist(rank, world, port)
    from moodist_b200.utils import selfcheck

    res = selfcheck.run_selfcheck(device="cpu")
    assert res["ok"] and res["cases"] == 12 and res["failed"] == [], res
    assert res["max_rel_err"] < 1e-2
    # a result that is off is caught and named
    ck = selfcheck._Checker(dist.group.WORLD, torch.device("cpu"))
    ck.compare("broken", torch.ones(8), torch.full((8,), 2.0), 1e-3)
    assert ck.failed and "broken" in ck.failed[0]
    dist.barrier()
    dist.destroy_process_group()


def test_selfcheck_on_cpu_ranks_world2():
    run_ranks(_body, 2, timeout=180)


def test_selfcheck_on_cpu_ranks_world3():
    run_ranks(_body, 3, timeout=240)
