"""Property tests (hypothesis) of the host runtime: the msgpack codec shared by Python and the
C++ servers, the consistent-hash ring, the byte-range file partitioner, the KV store and the
loader's binning of parsed lines.  The
reference tests these parts with fixed cases (test/test_packer.cpp, test_ring.cpp,
test_partition.cpp, test_kv.cpp); random inputs look for what those cases leave out."""
import os

import pytest
from hypothesis import HealthCheck, given, settings
from hypothesis import strategies as st

from paracel_b200._core import core
from paracel_b200.utils.packer import pack, unpack

_settings = settings(max_examples=150, deadline=None, derandomize=True,
                     suppress_health_check=[HealthCheck.function_scoped_fixture, HealthCheck.too_slow])

_scalars = st.one_of(st.booleans(), st.integers(-2 ** 62, 2 ** 62),
                     st.floats(allow_nan=False, allow_infinity=False, width=64),
                     st.text(max_size=12), st.none())
_values = st.recursive(
    _scalars,
    lambda inner: st.one_of(st.lists(inner, max_size=5),
                            st.dictionaries(st.text(max_size=6), inner, max_size=4)),
    max_leaves=12)


@_settings
@given(_values)
def test_codec_round_trip_of_nested_values(v):
    assert unpack(pack(v)) == v


@_settings
@given(st.lists(st.floats(-1e6, 1e6, allow_nan=False), min_size=1, max_size=40),
       st.lists(st.floats(-1e6, 1e6, allow_nan=False), min_size=1, max_size=40))
def test_native_add_handler_on_packed_vectors(a, b):
    """The servers apply handlers to packed bytes in C++: element-wise sum for equal lengths, an
    error (not a crash, not a silent truncation) otherwise."""
    c = core()
    if len(a) == len(b):
        out = unpack(c.apply_builtin_handler("add", pack(a), pack(b)))
        assert out == [x + y for x, y in zip(a, b)]
    else:
        with pytest.raises(RuntimeError):
            c.apply_builtin_handler("add", pack(a), pack(b))


@_settings
@given(st.sets(st.integers(0, 1000), min_size=2, max_size=8), st.lists(st.text(min_size=1, max_size=10), min_size=1, max_size=60),
       st.data())
def test_ring_moves_only_the_keys_of_a_removed_server(servers, keys, data):
    """Consistent hashing: taking one server out re-homes its keys and nobody else's; putting it
    back restores the original placement."""
    from paracel_b200.ps.ring import ring
    servers = sorted(servers)
    r = ring(servers)
    before = {k: r.get_server(k) for k in keys}
    assert set(before.values()) <= set(servers)
    gone = data.draw(st.sampled_from(servers))
    r.remove_server(gone)
    after = {k: r.get_server(k) for k in keys}
    for k in keys:
        if before[k] != gone:
            assert after[k] == before[k]
        else:
            assert after[k] != gone
    r.add_server(gone)
    assert {k: r.get_server(k) for k in keys} == before


@_settings
@given(st.lists(st.lists(st.text(alphabet="abcxyz0123456789,| :.", min_size=1, max_size=30), min_size=0, max_size=25),
                min_size=1, max_size=3),
       st.integers(1, 7), st.booleans())
def test_partition_gives_every_line_to_exactly_one_worker(tmp_path_factory, files, workers, trailing_newline):
    """Byte ranges over one or several files: the workers' line lists, concatenated in rank order,
    are the lines of the files in order, whatever the line lengths, the number of workers (more
    than lines included) and whether the last line ends with a newline."""
    from paracel_b200.load.partition import partition
    d = tmp_path_factory.mktemp("part")
    names, expected = [], []
    for n, lines in enumerate(files):
        p = os.path.join(str(d), f"f{n}.txt")
        body = "\n".join(lines)
        if lines and trailing_newline:
            body += "\n"
        with open(p, "w") as f:
            f.write(body)
        names.append(p)
        expected += [l for l in lines]
    part = partition(names, workers)
    part.files_partition()
    starts, ends = part.get_start_list(), part.get_end_list()
    assert len(starts) == len(ends)
    got = []
    for s, e in zip(starts, ends):
        got += part.files_load_lines_impl(s, e)
    # blank lines are not records
    assert got == [l for l in expected if l != ""]


class _KvModel:
    """What the store promises, on a plain dict."""

    def __init__(self):
        self.d = {}

    def apply(self, kv, op, key, val):
        if op == "set":
            kv.set(key, val)
            self.d[key] = val
        elif op == "incr":
            ok = kv.incr(key, val)
            want = key in self.d and isinstance(self.d[key], (int, float)) and not isinstance(self.d[key], bool)
            assert ok == want
            if want:
                self.d[key] += val
        elif op == "delete":
            assert kv.delete(key) == (key in self.d)
            self.d.pop(key, None)
        elif op == "cas":
            got = kv.gets(key)
            if key in self.d:
                cur, uniq = got
                assert cur == self.d[key]
                assert kv.cas(key, val, uniq)
                # the version token is a hash of the stored value (as in the reference): it stays
                # valid exactly when the write did not change the value
                again = kv.cas(key, val + 1, uniq)
                assert again == (val == cur)
                self.d[key] = val + 1 if again else val
            else:
                assert got is None


@_settings
@given(st.lists(st.tuples(st.sampled_from(["set", "incr", "delete", "cas"]), st.sampled_from(list("abcde")),
                          st.integers(-1000, 1000)), max_size=40))
def test_kv_store_against_a_dict_model(ops):
    from paracel_b200.ps.kv import kvs
    kv, model = kvs(), _KvModel()
    for op, key, val in ops:
        model.apply(kv, op, key, val)
        assert kv.contains(key) == (key in model.d)
    assert dict(kv.getall()) == model.d
    assert len(kv) == len(model.d)


_ids = st.integers(0, 500)
_edge = st.tuples(_ids, _ids, st.floats(0.125, 8.0, allow_nan=False))


@_settings
@given(st.lists(_edge, max_size=40), st.sampled_from(["fmap", "smap", "fsmap"]), st.sampled_from(["abw", "ab", "adj"]))
def test_lines_organize_bins_every_triple_where_h_says(edges, pattern, shape):
    """The loader's binning on a single rank with a pretend grid: each of the accepted line shapes
    (``a,b,w`` / ``a,b`` and ``a,b:w`` / adjacency lists with ``mix``) yields the same triples, each
    in the bin that ``h`` names for its endpoints, none lost and none doubled."""
    from paracel_b200.load.scheduler import scheduler
    from paracel_b200.parallel.comm import Comm
    from paracel_b200.utils.ext import str_split
    sch = scheduler(Comm(), pattern, mix=(shape == "adj"))
    sch.dim_init()
    if shape == "abw":
        lines = [f"{a},{b},{w!r}" for a, b, w in edges]
    elif shape == "ab":
        lines = [f"{a},{b}:{w!r}" if k % 2 else f"{a},{b}" for k, (a, b, w) in enumerate(edges)]
        edges = [(a, b, w if k % 2 else 1.0) for k, (a, b, w) in enumerate(edges)]
    else:
        by_src = {}
        for a, b, w in edges:
            by_src.setdefault(a, []).append((b, w))
        # an adjacency line needs at least two neighbours to be told from the "a,b" shape
        lines, kept = [], []
        for a, nb in by_src.items():
            if len(nb) < 2:
                continue
            lines.append(",".join([str(a)] + [f"{b}|{w!r}" for b, w in nb]))
            kept += [(a, b, w) for b, w in nb]
        edges = kept
    slots = sch.lines_organize(lines, lambda l: str_split(l, ","))
    assert len(slots) == 1
    got = [t for sl in slots for t in sl]
    assert sorted(got) == sorted((a, b, float(w)) for a, b, w in edges)
    for rank, sl in enumerate(slots):
        for a, b, _ in sl:
            assert sch.h(a, b) == rank


@_settings
@given(st.sampled_from(["", "W_", "usr_bias_", "x"]), st.sampled_from(["", "_pr", "_links"]),
       st.sets(st.integers(0, 2 ** 40), min_size=1, max_size=30), st.booleans(), st.data())
def test_key_directory_round_trip(prefix, suffix, ids, with_names, data):
    """String keys of a device table: ``key_of`` and ``row_of`` invert each other for every row,
    with and without original-id names; keys of other forms and ids outside the table map to
    nothing."""
    import numpy as np
    import torch
    from types import SimpleNamespace
    from paracel_b200.ps.device_store import TableEntry
    names = np.array(sorted(ids), dtype=np.int64) if with_names else None
    rows = len(ids) if with_names else data.draw(st.integers(1, 1000))
    e = TableEntry("rows", SimpleNamespace(rows=rows, width=4, device="cpu"), prefix=prefix, suffix=suffix,
                   names=names)
    probe = range(rows) if rows <= 50 else data.draw(st.lists(st.integers(0, rows - 1), min_size=1, max_size=20))
    for r in probe:
        k = e.key_of(r)
        assert k.startswith(prefix) and k.endswith(suffix)
        assert e.row_of(k) == r
    # an id that is not in the table
    outside = (max(ids) + 1) if with_names else rows
    assert e.row_of(f"{prefix}{outside}{suffix}") is None
    # another key form
    assert e.row_of(f"zz{prefix}0{suffix}") is None or prefix == ""
    if prefix or suffix:
        assert e.row_of("0") is None
    # the bulk form agrees with the scalar one
    if with_names:
        t = torch.as_tensor(names)
        assert e.rows_of_ids(t).tolist() == list(range(rows))
