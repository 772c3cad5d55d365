"""The allocation-free strided copy, called through its exported C symbol, against the regular
gather/scatter entry point run as a one-rank group.

Some callers of the kernel library may not allocate device memory (a plugin inside a server with a fixed
memory plan, a recovery or teardown path), so ``mb_strided_copy_noalloc`` keeps its piece table in a static
device array.  The test runs both entry
points on the same pieces, twice in a row (the second call reuses the array with a different table), and
expects bit-identical outputs: both are pure copies.  Collected last so that a failure here cannot hide
the result of any other test.
"""

import ctypes
import os

import pytest
import torch

pytestmark = pytest.mark.gpu

MAX_RANKS = 8


class Piece(ctypes.Structure):
    _fields_ = [
        ("src_rank", ctypes.c_int32),
        ("rows", ctypes.c_uint32),
        ("src_off", ctypes.c_uint64),
        ("src_local", ctypes.c_void_p),
        ("dst", ctypes.c_void_p),
        ("row_bytes", ctypes.c_uint64),
        ("src_pitch", ctypes.c_uint64),
        ("dst_pitch", ctypes.c_uint64),
    ]


class Comm(ctypes.Structure):
    _fields_ = [
        ("rank", ctypes.c_int),
        ("world", ctypes.c_int),
        ("peer", ctypes.c_void_p * MAX_RANKS),
        ("stage", ctypes.c_void_p * MAX_RANKS),
        ("flags", ctypes.c_void_p * MAX_RANKS),
        ("staging_bytes", ctypes.c_uint64),
        ("mc_stage", ctypes.c_void_p),
        ("mc_flags", ctypes.c_void_p),
        ("status", ctypes.c_void_p),
        ("wait_ns", ctypes.c_uint64),
        ("max_ctas", ctypes.c_int),
        ("tuning", ctypes.c_uint32),
    ]


def _lib():
    import moodist_b200  # noqa: F401 - makes sure the library is built and loadable
    from moodist_b200._core import LIB_PATH

    lib = ctypes.CDLL(LIB_PATH)
    lib.mb_strided_copy_noalloc.restype = ctypes.c_int
    lib.mb_strided_copy_noalloc.argtypes = [ctypes.POINTER(Piece), ctypes.c_int, ctypes.c_void_p]
    lib.mb_gather_scatter.restype = ctypes.c_int
    lib.mb_gather_scatter.argtypes = [ctypes.POINTER(Comm), ctypes.c_uint32, ctypes.c_void_p, ctypes.c_int, ctypes.c_void_p,
                                      ctypes.c_int, ctypes.c_size_t, ctypes.c_void_p]
    return lib


def _pieces(src, dst_a, dst_b, variant):
    """A row -> column style reshard of a [R, C] fp32 matrix plus one contiguous block."""
    R, C = src.shape
    es = src.element_size()
    half = C // 2
    specs = []
    # left half of every row -> rows of dst_a ([R, half]); right half -> dst_b, shifted by `variant` rows
    specs.append((src.data_ptr(), dst_a.data_ptr(), R, half * es, C * es, half * es))
    specs.append((src.data_ptr() + half * es, dst_b.data_ptr(), R - variant, half * es, C * es, half * es))
    # one contiguous piece: first row block of src into the tail of dst_b
    if variant:
        specs.append((src.data_ptr(), dst_b.data_ptr() + (R - variant) * half * es, 1, variant * half * es, variant * half * es,
                      variant * half * es))
    arr = (Piece * len(specs))()
    for p, (s, d, rows, rb, sp, dp) in zip(arr, specs):
        p.src_rank, p.rows, p.src_off, p.src_local, p.dst = 0, rows, 0, s, d
        p.row_bytes, p.src_pitch, p.dst_pitch = rb, sp, dp
    biggest = max(rows * rb for (_, _, rows, rb, _, _) in specs)
    return arr, biggest


def test_noalloc_strided_copy_matches_regular_entry_point():
    lib = _lib()
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(0)
    stream = torch.cuda.current_stream().cuda_stream
    # one-rank "group" for the regular entry point: a zeroed flag page and a status word are all it needs
    flags = torch.zeros(4096, dtype=torch.int32, device=dev)
    status = torch.zeros(16, dtype=torch.int32, device=dev)
    comm = Comm()
    comm.rank, comm.world = 0, 1
    comm.flags[0] = flags.data_ptr()
    comm.stage[0] = flags.data_ptr()
    comm.peer[0] = flags.data_ptr()
    comm.status = status.data_ptr()
    comm.wait_ns = 1_000_000_000
    R, C = 1024, 768
    for call, variant in enumerate((0, 5)):  # two calls in a row, second with a different table
        torch.manual_seed(call)
        src = torch.randn(R, C, device=dev)
        outs = []
        for which in ("noalloc", "regular"):
            dst_a = torch.full((R, C // 2), -1.0, device=dev)
            dst_b = torch.full((R, C // 2), -1.0, device=dev)
            arr, biggest = _pieces(src, dst_a, dst_b, variant)
            if which == "noalloc":
                rc = lib.mb_strided_copy_noalloc(arr, len(arr), stream)
            else:
                table = torch.frombuffer(bytearray(bytes(arr)), dtype=torch.uint8).to(dev)
                rc = lib.mb_gather_scatter(ctypes.byref(comm), call + 1, None, 0, table.data_ptr(), len(arr), biggest, stream)
            assert rc == 0, (which, rc)
            torch.cuda.synchronize()
            outs.append((dst_a.clone(), dst_b.clone()))
        assert int(status[0]) == 0
        (a0, b0), (a1, b1) = outs
        assert torch.equal(a0, a1) and torch.equal(b0, b1)
        assert torch.equal(a0, src[:, : C // 2])  # and both are right
        assert torch.equal(b0[: R - variant], src[: R - variant, C // 2:])
        if variant:
            assert torch.equal(b0[R - variant:].reshape(-1), src.reshape(-1)[: variant * (C // 2)])


def _fill(arr, specs):
    for p, (s, d, rows, rb, sp, dp) in zip(arr, specs):
        p.src_rank, p.rows, p.src_off, p.src_local, p.dst = 0, rows, 0, s, d
        p.row_bytes, p.src_pitch, p.dst_pitch = rb, sp, dp


def test_noalloc_unaligned_pieces_and_full_table():
    """Pieces off every 16-byte boundary (odd row length, odd pitches, source pointer moved by three bytes,
    an empty piece), then a call that fills the table to its last slot."""
    lib = _lib()
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(0)
    stream = torch.cuda.current_stream().cuda_stream
    g = torch.Generator().manual_seed(11)
    src = torch.randint(0, 256, (400_000,), generator=g, dtype=torch.uint8).to(dev)  # 4096 x 96 bytes fit
    dst = torch.zeros(200_000, dtype=torch.uint8, device=dev)
    rows, rb, sp, dp = 37, 1003, 2011, 1005
    specs = [
        (src.data_ptr() + 3, dst.data_ptr() + 1, rows, rb, sp, dp),          # strided, nothing aligned
        (src.data_ptr() + 100_001, dst.data_ptr() + 100_003, 1, 12_345, 12_345, 12_345),  # contiguous, unaligned
        (src.data_ptr(), dst.data_ptr() + 199_000, 0, 64, 64, 64),           # no rows: copies nothing
    ]
    arr = (Piece * len(specs))()
    _fill(arr, specs)
    assert lib.mb_strided_copy_noalloc(arr, len(arr), stream) == 0
    torch.cuda.synchronize()
    s_host, d_host = src.cpu(), dst.cpu()
    want = torch.zeros(200_000, dtype=torch.uint8)
    for r in range(rows):
        want[1 + r * dp : 1 + r * dp + rb] = s_host[3 + r * sp : 3 + r * sp + rb]
    want[100_003 : 100_003 + 12_345] = s_host[100_001 : 100_001 + 12_345]
    assert torch.equal(d_host, want)
    # exactly MB_NOALLOC_MAX_PIECES pieces of 48 bytes each: a gather of every other 48-byte block
    n = 4096
    dst2 = torch.zeros(n * 48, dtype=torch.uint8, device=dev)
    specs = [(src.data_ptr() + i * 96, dst2.data_ptr() + i * 48, 1, 48, 48, 48) for i in range(n)]
    arr = (Piece * n)()
    _fill(arr, specs)
    assert lib.mb_strided_copy_noalloc(arr, n, stream) == 0
    torch.cuda.synchronize()
    assert torch.equal(dst2.cpu().view(n, 48), s_host[: n * 96].view(n, 96)[:, :48])


def test_noalloc_rejects_oversized_tables():
    lib = _lib()
    torch.cuda.set_device(0)
    arr = (Piece * 4097)()
    assert lib.mb_strided_copy_noalloc(arr, 4097, None) == 5  # MB_ERR_TOO_BIG, nothing launched
    assert lib.mb_strided_copy_noalloc(arr, -1, None) == 1
