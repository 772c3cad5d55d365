"""Per-group options, the prefer_kernel_less context, group lookup by name and the default switch, on CPU ranks."""

import pytest
import torch

from moodist_b200.utils.testing import init_moodist, run_ranks


def _options(rank, world, port):
    dist = init_moodist(rank, world, port)
    import moodist_b200 as moodist

    pg = moodist.get_backend(device="cpu")
    assert moodist.find_process_group(pg.moodist_name()) is not None
    assert moodist.find_process_group("no-such-group") is None
    names = [None] * world
    dist.all_gather_object(names, pg.moodist_name())
    assert len(set(names)) == 1, "every rank sees the same group name"

    opts = pg.options()
    assert opts.method is None and opts.num_chunks is None and opts.prefer_kernel_less is False
    opts.method = 1
    opts.num_chunks = 4
    assert opts.method == 1 and opts.num_chunks == 4
    with pg.options(method=0, prefer_kernel_less=True) as same:
        assert same is pg
        assert pg.options().method == 0 and pg.options().prefer_kernel_less is True
        t = torch.ones(10)
        dist.all_reduce(t)  # CPU collectives do not care about the CUDA variant options
        assert bool((t == world).all())
    assert pg.options().method == 1 and pg.options().prefer_kernel_less is False
    opts.method = None
    assert pg._get_option("method") == -1
    with pytest.raises(AttributeError):
        opts.no_such_option = 1
    with pytest.raises(AttributeError):
        _ = opts.no_such_option
    with pytest.raises(ValueError):
        pg.options(bogus=1)

    assert pg.get_prefer_kernel_less() is False
    with pg.prefer_kernel_less(True):
        assert pg.get_prefer_kernel_less() is True
    assert pg.get_prefer_kernel_less() is False
    ctx = moodist.PreferKernelLessContext(pg, True)  # takes effect at construction, like the reference's
    assert pg.get_prefer_kernel_less() is True
    ctx.__exit__(None, None, None)
    assert pg.get_prefer_kernel_less() is False
    assert isinstance(pg.describe(), str) and pg.kernel_launches() == 0
    dist.barrier()
    dist.destroy_process_group()


def test_options_and_lookup():
    run_ranks(_options, 2, timeout=120)
