"""CPU ranks on one machine move payloads with one process_vm_readv copy instead of a loopback socket; where
the kernel refuses (or MOODIST_DIRECT_CPU=0 says so) everything stays on TCP.  Both paths give the oracle's
results; the traffic counters tell which one ran."""

import torch

from moodist_b200.utils.testing import init_moodist, run_ranks


def _body(rank, world, port, direct_wanted):
    dist = init_moodist(rank, world, port)
    import moodist_b200

    pg = moodist_b200.get_backend(device="cpu")
    n = 300_000
    g = torch.Generator().manual_seed(0)
    full = torch.randn(world, n, generator=g)
    dist.barrier()
    start = pg.host_stats()
    for _ in range(2):
        x = full[rank].clone()
        dist.all_reduce(x)
        torch.testing.assert_close(x, full.sum(0), rtol=1e-5, atol=1e-5)
        out = torch.empty(world * n)
        dist.all_gather_into_tensor(out, full[rank].clone())
        assert torch.equal(out.view(world, n), full)
        o = torch.empty(n // world)
        dist.reduce_scatter_tensor(o, full[rank, : (n // world) * world].clone(), op=dist.ReduceOp.AVG)
        want = full[:, : (n // world) * world].view(world, world, -1)[:, rank].mean(0)
        torch.testing.assert_close(o, want, rtol=1e-5, atol=1e-6)
        b = full[rank].clone()
        dist.broadcast(b, src=world - 1)
        assert torch.equal(b, full[world - 1])
    # one-sided strided reads: a row -> column reshard through compile_op
    m = 256 * world
    gm = torch.randn(m, m, generator=torch.Generator().manual_seed(1))
    rows = m // world
    op = moodist_b200.compile_op(pg, shape=(m, m), dtype=torch.float32,
                                 inputs=[{"offset": [rank * rows, 0], "shape": [rows, m]}],
                                 outputs=[{"offset": [0, rank * rows], "shape": [m, rows]}])
    dst = torch.empty(m, rows)
    op([gm[rank * rows : (rank + 1) * rows].contiguous()], [dst]).wait()
    assert torch.equal(dst, gm[:, rank * rows : (rank + 1) * rows])
    # a queue item too large to travel inside its message is fetched with a one-sided read
    q = moodist_b200.Queue(pg, location=0, name="direct-test")
    if rank == world - 1:
        q.put_tensor(full[rank]).wait()
    dist.barrier()
    if rank == 0:
        assert torch.equal(q.get_tensor(timeout=30), full[world - 1])
    dist.barrier()
    end = pg.host_stats()
    direct = end["direct_bytes"] - start["direct_bytes"]
    tcp = end["tcp_bytes_received"] - start["tcp_bytes_received"]
    if not direct_wanted:
        assert end["direct_peers"] == 0 and direct == 0 and tcp > 4 * n, end
    elif end["direct_peers"] > 0:
        # payloads bypassed the sockets: what is left on them is headers, announcements and completions
        assert direct > 4 * n and tcp < direct / 20, (start, end)
    else:
        assert direct == 0 and tcp > 4 * n, end  # this machine does not allow it: the fallback carried everything
    dist.barrier()
    dist.destroy_process_group()


def test_direct_copies_between_cpu_ranks_world2():
    run_ranks(_body, 2, True, timeout=180)


def test_direct_copies_between_cpu_ranks_world3():
    run_ranks(_body, 3, True, timeout=180)


def test_forced_tcp_fallback():
    run_ranks(_body, 2, False, timeout=180, env={"MOODIST_DIRECT_CPU": 0})


def test_plain_tcp_as_between_machines():
    """Neither same-machine shortcut: every byte over loopback TCP, the path ranks on different hosts take."""
    run_ranks(_body, 3, False, timeout=180, env={"MOODIST_DIRECT_CPU": 0, "MOODIST_DISABLE_UNIX_SOCKETS": 1})


def _sockets(rank, world, port, unix_wanted):
    dist = init_moodist(rank, world, port)
    import moodist_b200

    pg = moodist_b200.get_backend(device="cpu")
    x = torch.full((1000,), float(rank + 1))
    dist.all_reduce(x)
    assert float(x[0]) == world * (world + 1) / 2
    stats = pg.host_stats()
    # ranks of one machine reach each other over unix-domain sockets unless that is switched off, in which case
    # the TCP addresses advertised after it are used
    assert stats["unix_socket_peers"] == (world - 1 if unix_wanted else 0), stats
    dist.barrier()
    dist.destroy_process_group()


def test_same_machine_ranks_use_unix_sockets():
    run_ranks(_sockets, 3, True, timeout=120)


def test_tcp_when_unix_sockets_are_off():
    run_ranks(_sockets, 2, False, timeout=120, env={"MOODIST_DISABLE_UNIX_SOCKETS": 1})
