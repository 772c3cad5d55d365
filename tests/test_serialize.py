"""Python-object serializer: golden bytes of the wire format plus round trips, following the cases of
the reference's tests/test_serialize.py (every tag, big ints, special floats, UCS kinds, shared and
circular references, functions, types, custom __reduce__, numpy arrays)."""

import collections
import dataclasses
import enum
import math
import struct

import pytest
import torch

import moodist_b200 as moodist


def pack(obj) -> bytes:
    t = moodist.serialize(obj)
    assert isinstance(t, torch.Tensor) and t.dtype == torch.uint8 and t.dim() == 1
    return bytes(t.numpy())


def roundtrip(obj):
    return moodist.deserialize(moodist.serialize(obj))


GOLDEN = [
    (None, "00"),
    (True, "01"),
    (False, "02"),
    (0, "0300"),
    (-1, "03ff"),
    (127, "037f"),
    (128, "048000"),
    (-129, "047fff"),
    (70000, "0570110100"),
    (2**30 - 1, "05ffffff3f"),
    (1.5, "07" + struct.pack("<d", 1.5).hex()),
    ("a", "0d01" + "0100000000000000" + "61"),
    ("é", "0d01" + "0100000000000000" + "e9"),
    ("中", "0d02" + "0200000000000000" + "2d4e"),
    ("\U0001f600", "0d04" + "0400000000000000" + "00f60100"),
    (b"xy", "0e" + "0200000000000000" + "7879"),
    (bytearray(b"z"), "0f" + "0100000000000000" + "7a"),
    ([], "0a0300"),
    ([1, 300, "a", None], "0a0304" + "0301" + "042c01" + "0d01010000000000000061" + "00"),
    ((1, 2), "0b0302" + "0301" + "0302"),
    ({"k": 1}, "080301" + "0d0101000000000000006b" + "0301"),
    ({5}, "10" + "0100000000000000" + "0305"),
    (frozenset({5}), "11" + "0100000000000000" + "0305"),
    # ints that CPython does not store compactly (>= 2**30) travel as bigint: u64 count + LE two's complement
    (2**30, "0c" + "0500000000000000" + "0000004000"),
    (2**64, "0c" + "0a00000000000000" + "00" * 8 + "0100"),
    (len, "12" + "0d0103000000000000006c656e" + "0d01" + "0800000000000000" + b"builtins".hex()),
]


@pytest.mark.parametrize("obj,hexbytes", GOLDEN, ids=[repr(g[0])[:20] for g in GOLDEN])
def test_golden_bytes(obj, hexbytes):
    assert pack(obj).hex() == hexbytes
    assert roundtrip(obj) == obj


def test_shared_reference_marks_original_tag():
    shared = [7]
    data = pack([shared, shared])
    # outer list @0, first inner list @3 gets 0x80, second occurrence is `offset` (tag 20) + u64 3
    assert data.hex() == "0a0302" + "8a03010307" + "14" + "0300000000000000"
    r = roundtrip([shared, shared])
    assert r[0] is r[1] and r[0] == [7]


def test_circular_reference():
    l = [1, 2]
    l.append(l)
    r = roundtrip(l)
    assert r[0] == 1 and r[2] is r
    d = {}
    d["self"] = d
    r = roundtrip(d)
    assert r["self"] is r


class _Pair:
    def __init__(self):
        self.a = self.b = None


class _HashableHolder:
    held = None

    def __hash__(self):
        return 7


def test_tuples_that_contain_themselves_keep_their_identity():
    # the writer refers to the tuple from inside its own members; the reader hands a referenced tuple out before
    # it is whole, as it does with a list (and as the reference's reader does)
    inner = []  # a single reference: not in the writer's memo
    t = (inner,)
    inner.extend([t, t])
    r = roundtrip(t)
    assert r[0][0] is r and r[0][1] is r and len(r) == 1 and len(r[0]) == 2
    import gc

    assert gc.is_tracked(r)  # it is part of a cycle, so the collector must see it
    shared = []
    t = (shared, "x")
    shared.append(t)
    r = roundtrip([t, t, shared])
    assert r[0] is r[1] and r[2][0] is r[0] and r[0][0] is r[2] and r[0][1] == "x"
    node = _Pair()
    node.a = (node, {"back": node})
    node.b = node.a
    r = roundtrip(node)
    assert r.a is r.b and r.a[0] is r and r.a[1]["back"] is r
    # a frozenset has no such early form: refused when writing, not when some other rank reads
    holder = _HashableHolder()
    holder.held = frozenset([holder, 1])
    with pytest.raises(ValueError, match="frozenset that contains itself"):
        pack([holder.held])
    assert roundtrip([frozenset([1, 2]), frozenset([1, 2])]) == [frozenset([1, 2])] * 2


def _random_graph(rng, n):
    nodes = []
    for _ in range(n):
        kind = rng.choice(["list", "dict", "pair", "frozenset", "bytes", "str", "int", "float", "tuple"])
        if kind == "list":
            nodes.append([])
        elif kind == "dict":
            nodes.append({})
        elif kind == "pair":
            nodes.append(_Pair())
        elif kind == "frozenset":
            nodes.append(frozenset(rng.sample(range(100), rng.randint(0, 4))))
        elif kind == "bytes":
            nodes.append(bytes(rng.randrange(256) for _ in range(rng.randint(0, 300))))
        elif kind == "str":
            nodes.append("s" * rng.randint(0, 5) + str(rng.random()))
        elif kind == "int":
            nodes.append(rng.choice([0, -1, 2**31, 2**63, -(2**64), 10**40, rng.randrange(1000)]))
        elif kind == "float":
            nodes.append(rng.random())
        else:  # tuples of earlier nodes: they get into cycles through the lists, dicts and pairs filled below
            nodes.append(tuple(rng.choice(nodes) for _ in range(rng.randint(0, 3))) if nodes else ())
    for node in nodes:
        if isinstance(node, list):
            node.extend(rng.choice(nodes) for _ in range(rng.randint(0, 5)))
        elif isinstance(node, dict):
            for _ in range(rng.randint(0, 4)):
                node[rng.choice(["k1", "k2", 3, (1, 2), 4.5, b"z"])] = rng.choice(nodes)
        elif isinstance(node, _Pair):
            node.a, node.b = rng.choice(nodes), rng.choice(nodes)
    return [nodes[0], nodes[-1], nodes]


def _shape_with_identities(root):
    """The graph as a flat list in traversal order; a container met again appears as the number of its first visit."""
    seen, out, todo = {}, [], [root]
    while todo:
        o = todo.pop()
        if isinstance(o, (list, dict, _Pair, tuple)):
            if id(o) in seen:
                out.append(("again", seen[id(o)]))
                continue
            seen[id(o)] = len(seen)
        if isinstance(o, (list, tuple)):
            out.append((type(o).__name__, len(o)))
            todo.extend(reversed(o))
        elif isinstance(o, dict):
            out.append(("dict", list(o)))
            todo.extend(reversed(list(o.values())))
        elif isinstance(o, _Pair):
            out.append(("pair",))
            todo.extend([o.b, o.a])
        else:
            out.append((type(o).__name__, o))
    return out


def test_random_object_graphs_with_shared_members_and_cycles():
    import random

    deep = 0
    for seed in range(300):
        rng = random.Random(seed)
        graph = _random_graph(rng, rng.randint(1, 60))
        try:
            back = roundtrip(graph)
        except RecursionError:  # a chain deeper than the writer's limit: refused, which is fine
            deep += 1
            continue
        assert _shape_with_identities(back) == _shape_with_identities(graph), seed
    assert deep < 30


def test_scalars_and_special_floats():
    for v in (0, 1, -1, 2**7, -(2**7), 2**15, -(2**15) - 1, 2**31, -(2**31) - 1, 2**62, 2**63, -(2**63), 2**200, -(2**200)):
        assert roundtrip(v) == v
    assert roundtrip(float("inf")) == float("inf")
    assert roundtrip(float("-inf")) == float("-inf")
    assert math.isnan(roundtrip(float("nan")))
    assert math.copysign(1, roundtrip(-0.0)) == -1


def test_containers_nested():
    obj = {"a": [1, (2, 3), {"b": {4, 5}}], "c": frozenset({6}), 7: None, (8, 9): b"ten", "e": bytearray(b"11")}
    assert roundtrip(obj) == obj
    big = list(range(-1000, 1000))
    assert roundtrip(big) == big


def top_level_function(x):
    return x + 1


class Point:
    def __init__(self, x, y):
        self.x, self.y = x, y

    def __eq__(self, o):
        return type(o) is Point and (o.x, o.y) == (self.x, self.y)


class WithReduce:
    def __init__(self, v):
        self.v = v

    def __reduce__(self):
        return (WithReduce, (self.v * 2,))


class WithSlots:
    __slots__ = ("a", "b")

    def __init__(self):
        self.a, self.b = 1, [2]


def test_functions_types_and_objects():
    assert roundtrip(top_level_function) is top_level_function
    assert roundtrip(Point) is Point
    assert roundtrip(collections.OrderedDict) is collections.OrderedDict
    assert roundtrip(Point(1, [2, 3])) == Point(1, [2, 3])
    assert roundtrip(WithReduce(21)).v == 42
    s = roundtrip(WithSlots())
    assert s.a == 1 and s.b == [2]
    od = collections.OrderedDict(a=1, b=2)
    r = roundtrip(od)
    assert r == od and type(r) is collections.OrderedDict
    dd = collections.defaultdict(list)
    dd["k"].append(1)
    r = roundtrip(dd)
    assert r == dd and r.default_factory is list
    dq = collections.deque([1, 2, 3], maxlen=5)
    r = roundtrip(dq)
    assert r == dq and r.maxlen == 5


class Colour(enum.Enum):
    RED = 1
    BLUE = 2


@dataclasses.dataclass(frozen=True, slots=True)
class FrozenRecord:
    x: int
    y: str


class KeepsOnlyX:
    def __init__(self):
        self.x, self.cache = 1, "computed"

    def __getstate__(self):
        return {"x": self.x}

    def __setstate__(self, state):
        self.x, self.cache = state["x"], "rebuilt"


Pair = collections.namedtuple("Pair", "a b")


def test_standard_library_objects_follow_pickle():
    """Objects whose way back is described by __reduce_ex__, __getstate__, copyreg or a bare global name."""
    import datetime
    import decimal
    import fractions
    import functools
    import pathlib
    import re
    import uuid

    plain = [
        Colour.BLUE, FrozenRecord(3, "z"), Pair(1, Pair(2, 3)),
        datetime.datetime(2024, 1, 2, 3, 4, 5, 6), datetime.date(2020, 2, 29), datetime.timedelta(days=1, microseconds=5),
        datetime.timezone.utc, decimal.Decimal("1.2345"), fractions.Fraction(3, 7), 1 + 2j,
        pathlib.PurePosixPath("/a/b"), uuid.UUID(int=5), range(1, 10, 2), slice(1, 2, 3),
        collections.Counter("hello"), frozenset({(1, 2), (3, 4)}), 2**200, -(2**200),
    ]
    for obj in plain:
        back = roundtrip(obj)
        assert back == obj and type(back) is type(obj), obj
    assert roundtrip(Colour.RED) is Colour.RED
    # singletons that pickle stores as a bare name; they have no __module__ of their own
    assert roundtrip([Ellipsis, NotImplemented]) == [Ellipsis, NotImplemented]
    # a reducer registered through copyreg (how compiled regular expressions travel)
    pattern = roundtrip(re.compile(r"a+b", re.I))
    assert pattern.pattern == "a+b" and pattern.flags == re.compile(r"a+b", re.I).flags and pattern.match("AAB")
    part = roundtrip(functools.partial(int, base=2))
    assert part("101") == 5
    state = roundtrip(KeepsOnlyX())
    assert state.x == 1 and state.cache == "rebuilt"


def test_objects_that_cannot_be_found_again_are_refused_when_serializing():
    """A lambda or a class made inside a function has no importable name: like pickle, say so on the sending
    side instead of failing on the receiving one."""

    class Local:
        pass

    for obj in (lambda x: x, Local, Local()):
        with pytest.raises(ValueError, match="cannot serialize"):
            moodist.serialize(obj)
    for obj in ((i for i in range(3)), collections, open(__file__)):
        with pytest.raises(TypeError):
            moodist.serialize(obj)


def test_numpy_and_torch_payloads():
    np = pytest.importorskip("numpy")
    a = np.arange(12.0).reshape(3, 4)
    r = roundtrip(a)
    assert isinstance(r, np.ndarray) and (r == a).all() and r.dtype == a.dtype
    t = torch.arange(6.0).view(2, 3)
    assert torch.equal(roundtrip(t), t)


def test_errors():
    with pytest.raises(ValueError):
        moodist.deserialize(torch.tensor([10, 3, 5, 3], dtype=torch.uint8))  # list of 5 but truncated
    with pytest.raises(ValueError):
        moodist.deserialize(torch.tensor([99], dtype=torch.uint8))  # unknown tag
    with pytest.raises(ValueError):
        moodist.deserialize(torch.tensor([0, 0], dtype=torch.uint8))  # trailing bytes
    with pytest.raises(TypeError):
        moodist.deserialize(torch.zeros(2))


def test_roundtrip_property_based():
    """Randomly generated nested objects survive serialize -> deserialize unchanged, shared references stay shared."""
    from hypothesis import given, settings
    from hypothesis import strategies as st

    import moodist_b200 as moodist

    scalars = st.one_of(
        st.none(), st.booleans(), st.integers(min_value=-(2**80), max_value=2**80),
        st.floats(allow_nan=False), st.text(max_size=40), st.binary(max_size=40),
    )
    hashable = st.one_of(st.integers(), st.text(max_size=10), st.booleans(), st.none(),
                         st.tuples(st.integers(), st.text(max_size=5)))
    objects = st.recursive(
        scalars,
        lambda inner: st.one_of(
            st.lists(inner, max_size=6), st.tuples(inner, inner), st.dictionaries(hashable, inner, max_size=6),
            st.frozensets(hashable, max_size=5), st.sets(hashable, max_size=5),
        ),
        max_leaves=40,
    )

    @settings(max_examples=300, deadline=None)
    @given(objects)
    def check(obj):
        back = moodist.deserialize(moodist.serialize(obj))
        assert back == obj and type(back) is type(obj)
        shared = [obj, obj, (obj,)]
        b2 = moodist.deserialize(moodist.serialize(shared))
        assert b2 == shared
        if isinstance(obj, (list, dict, set)):
            assert b2[0] is b2[1] and b2[2][0] is b2[0]

    check()


def test_truncated_and_corrupt_input_raise():
    """Every prefix of a valid encoding and random byte flips either raise a Python exception or decode to some
    object; none may crash the process."""
    import random

    import moodist_b200 as moodist

    obj = {"a": [1, 2.5, "x" * 20, b"bytes", (None, True)], "b": {1, 2, 3}, "c": 2**70, "d": [[], {}, ()]}
    blob = bytes(moodist.serialize(obj).numpy().tobytes() if hasattr(moodist.serialize(obj), "numpy") else moodist.serialize(obj))
    for cut in range(len(blob)):
        try:
            moodist.deserialize(blob[:cut])
        except Exception:
            pass
    rng = random.Random(0)
    for _ in range(500):
        b = bytearray(blob)
        for _ in range(rng.randint(1, 3)):
            b[rng.randrange(len(b))] = rng.randrange(256)
        try:
            moodist.deserialize(bytes(b))
        except Exception:
            pass
    # the same for streams with objects rebuilt through callables, back references and lists that contain
    # themselves: damage there can point a reference at a container that is still being filled, or put
    # something that is not a list where list items are expected
    shared = [1, 2, 3]
    cyclic = [shared, shared, {"again": shared}]
    cyclic.append(cyclic)
    rich = [Point(1, [2, 3]), WithSlots(), collections.OrderedDict(a=1), collections.deque([1, 2], maxlen=4), cyclic,
            collections.defaultdict(list, {"k": [1]}), Colour.RED, FrozenRecord(1, "y"), frozenset({(1, 2)})]
    blob = bytes(moodist.serialize(rich).numpy().tobytes())
    assert moodist.deserialize(blob)[0] == Point(1, [2, 3])
    for cut in range(len(blob)):
        try:
            moodist.deserialize(blob[:cut])
        except Exception:
            pass
    for _ in range(4000):
        b = bytearray(blob)
        for _ in range(rng.randint(1, 3)):
            b[rng.randrange(len(b))] = rng.randrange(256)
        try:
            moodist.deserialize(bytes(b))
        except Exception:
            pass
