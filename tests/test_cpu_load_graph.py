"""Partitioner, parsers, scheduler placement, graph containers (cases of the reference's
test_partition.cpp and test_graph.cpp plus the loader paths)."""

import numpy as np
import pytest

from paracel_b200.graph import (BFS, DFS, bigraph, bigraph_continuous, connected_components, digraph,
                                undirected_graph)
from paracel_b200.load.loader import loader
from paracel_b200.load.parser import gen_parser, parser_a, parser_a_int, parser_b
from paracel_b200.load.partition import partition
from paracel_b200.load.scheduler import scheduler
from paracel_b200.parallel.comm import Comm
from paracel_b200.utils.packer import pack, unpack


def _write(tmp_path, name, lines, trailing_newline=True):
    p = tmp_path / name
    p.write_text("\n".join(lines) + ("\n" if trailing_newline else ""))
    return str(p)


def test_partition_never_loses_or_duplicates_lines(tmp_path):
    rng = np.random.default_rng(0)
    lines_a = ["%d %s" % (i, "x" * int(rng.integers(0, 40))) for i in range(300)]
    lines_b = ["b%d,%d" % (i, i * i) for i in range(157)]
    fa = _write(tmp_path, "a.txt", lines_a)
    fb = _write(tmp_path, "b.txt", lines_b, trailing_newline=False)
    single = str(tmp_path / "ab.txt")
    open(single, "w").write(open(fa).read() + open(fb).read() + "\n")
    for np_ in range(1, 100):
        for names, expect in (([fa, fb], lines_a + lines_b), ([single], lines_a + lines_b)):
            for pattern in ("linesplit", "fmap"):
                if pattern == "fmap" and np_ > 12:
                    continue
                p = partition(names, np_, pattern)
                p.files_partition()
                ss, ee = p.get_start_list(), p.get_end_list()
                assert len(ss) == np_ * (1 if pattern == "linesplit" else 32)
                assert ss[0] == 0 and all(ee[i] == ss[i + 1] for i in range(len(ss) - 1))
                got = []
                for s, e in zip(ss, ee):
                    got.extend(p.files_load_lines_impl(s, e))
                assert got == expect, (np_, pattern, len(names))


def test_single_file_partition_helper(tmp_path):
    f = _write(tmp_path, "x.txt", ["l%d" % i for i in range(50)])
    p = partition([f], 7)
    ss, ee = p.file_partition(f)
    got = []
    for s, e in zip(ss, ee):
        got.extend(p.file_load_lines_impl(f, s, e))
    assert got == ["l%d" % i for i in range(50)]


def test_crlf_and_empty_lines(tmp_path):
    p = tmp_path / "c.txt"
    p.write_bytes(b"a,1\r\n\r\nb,2\r\nc,3")
    part = partition([str(p)], 1)
    part.files_partition()
    assert part.files_load_lines_impl(0, part.get_end_list()[-1]) == ["a,1", "", "b,2", "c,3"]


def test_parsers():
    assert parser_a("a b c d") == ["a", "b", "c", "d"]
    assert parser_a_int("1 2 3") == [1, 2, 3]
    assert parser_b("a b|c|d", " ", "|") == ["a", "b", "c", "d"]
    assert parser_b("a\tb:0.1 c:0.2", "\t") == ["a", "b:0.1", "c:0.2"]
    assert gen_parser(parser_a, ",")("x,y") == ["x", "y"]
    assert gen_parser(parser_b, " ", "|")("a b:0.1|c:0.2") == ["a", "b:0.1", "c:0.2"]


def test_lines_organize_shapes():
    sch = scheduler(Comm(), "fmap", mix=False)
    assert sch.lines_organize(["1 2", "3 4:0.5", "5 6 0.25"], parser_a)[0] == \
        [(1, 2, 1.0), (3, 4, 0.5), (5, 6, 0.25)]
    schm = scheduler(Comm(), "fmap", mix=True)
    assert schm.lines_organize(["1 2 3", "4 5|0.2 6|0.4"], parser_a)[0] == \
        [(1, 2, 1.0), (1, 3, 1.0), (4, 5, 0.2), (4, 6, 0.4)]
    with pytest.raises(ValueError):
        sch.lines_organize(["1 2 3 4"], parser_a)
    s = sch.lines_organize(["a b 2.0"], parser_a, numeric=False)
    assert s[0] == [("a", "b", 2.0)]
    # native numeric organiser agrees, including the slot (a % npx) * npy + b % npy
    from paracel_b200._core import core
    a, b, w, slot = core().organize_numeric([["7", "9", "1.5"], ["2", "4:0.5"]], False, 2, 2)
    assert a.tolist() == [7, 2] and b.tolist() == [9, 4] and w.tolist() == [1.5, 0.5]
    assert slot.tolist() == [(7 % 2) * 2 + 9 % 2, (2 % 2) * 2 + 4 % 2]
    sch2 = scheduler(Comm(), "fsmap")
    assert sch2.h(7, 9, 2, 2) == 3 and sch2.select(5) == 0


def test_loader_single_rank_graphs_and_matrices(tmp_path):
    f = _write(tmp_path, "g.txt", ["1,2,0.5", "1,3,1.5", "2,3,2.0", "7,1,1.0"])
    ld = loader(f, Comm(), gen_parser(parser_a, ","), "fmap")
    lines = ld.fixload()
    assert len(lines) == 4 and ld.load() == lines
    g = digraph()
    ld.create_graph(lines, g)
    assert g.e() == 4 and g.outdegree(1) == 2 and g.indegree(3) == 2 and g.reverse_adjacent(3) == {1: 1.5, 2: 2.0}
    bg = bigraph()
    ld.create_graph(lines, bg)
    assert bg.v() == 3 and bg.get_wgt(7, 1) == 1.0 and bg.is_connected(1, 2) and not bg.is_connected(2, 1)
    bc = bigraph_continuous()
    rm, cm = ld.create_graph(lines, bc)
    assert rm == {0: 1, 1: 2, 2: 7} and cm == {0: 1, 1: 2, 2: 3} and bc.e() == 4 and bc.outdegree(0) == 2
    blk, rm2, cm2 = ld.create_matrix(lines)
    assert blk.shape == (3, 3) and blk[0, 2] == 1.5 and blk[2, 0] == 1.0
    fd = _write(tmp_path, "d.txt", ["u1,0.5,1.5", "u2,2.5,3.5"])
    m, rmap = loader(fd, Comm(), gen_parser(parser_a, ","), "fvec").create_matrix(
        open(fd).read().split("\n"), dense=True, numeric=False)
    assert m.tolist() == [[0.5, 1.5], [2.5, 3.5]] and rmap == {0: "u1", 1: "u2"}
    seen = []
    ld.fixload_handle(seen.append)
    assert seen == lines
    # native triple loader straight from the byte ranges
    p = partition([f], 1, "fmap")
    p.files_partition()
    a, b, w, slot = p.native().load_triples(0, 32, ",", False, 1, 1, [])
    assert a.tolist() == [1, 1, 2, 7] and w.tolist() == [0.5, 1.5, 2.0, 1.0]


def test_graph_containers():
    ug = undirected_graph([(0, 5), (4, 3), (0, 1), (9, 12), (6, 4), (5, 4), (0, 2), (11, 12), (9, 10),
                           (0, 6), (7, 8), (9, 11), (5, 3)])
    assert ug.v() == 13 and ug.e() == 13 and ug.degree(0) == 4 and ug.max_degree() == 4
    assert ug.selfloops() == 0 and set(ug.adjacent(9)) == {10, 11, 12}
    assert abs(ug.avg_degree() - 1.0) < 1e-9
    cc = connected_components(ug)
    assert cc.cnt() == 3 and cc.is_connected(0, 3) and not cc.is_connected(0, 7) and cc.id(99) == -1
    order = []
    d = DFS(ug, 0, order.append)
    assert order[0] == 0 and set(order) == {0, 1, 2, 3, 4, 5, 6} and d.visited(4) and not d.visited(9)
    b = BFS(ug, 0)
    assert b.dist(0) == 0 and b.dist(3) == 2 and b.edgeTo(3) in (5, 4) and not b.visited(7)
    dg = digraph({"a": {"b": 1.0, "c": 2.0}, "b": {"c": 3.0}})
    assert dg.v() == 3 and dg.e() == 3 and dg.outdegree("a") == 2 and dg.indegree("c") == 2
    assert sorted(dg.dump2triples()) == [("a", "b", 1.0), ("a", "c", 2.0), ("b", "c", 3.0)]
    dg.reverse()
    assert dg.adjacent("c") == {"a": 2.0, "b": 3.0}
    dg.reverse()
    seen = []
    dg.traverse(lambda v, w, x: seen.append((v, w, x)))
    assert len(seen) == 3
    dg.traverse("a", lambda v, w, x: seen.append(("only", w)))
    assert ("only", "b") in seen
    topo = DFS(dg, "a").torder()
    assert topo.index("a") < topo.index("b") < topo.index("c")
    bg = bigraph([(1, 10, 3.0), (1, 11, 4.0), (2, 10, 5.0)])
    assert bg.left_vertex_set() == {1, 2} and bg.indegree(10) == 2 and bg.dump2dict() == {1: {10: 3.0, 11: 4.0}, 2: {10: 5.0}}
    src, dst, w = bg.to_coo()
    assert src.tolist() == [1, 1, 2] and w.tolist() == [3.0, 4.0, 5.0]
    bg.clear()
    assert bg.v() == 0 and bg.e() == 0
    # graphs are packable parameter values
    for g in (ug, dg, bigraph([(1, 2, 0.5)])):
        g2 = type(g).from_packable(unpack(pack(g)))
        assert g2.dump2dict() == g.dump2dict() and g2.e() == g.e()
    bc = bigraph_continuous(3)
    bc.add_edge(0, 7, 1.0)
    bc.add_edge(5, 1, 2.0)
    assert bc.v() == 6 and bc.e() == 2 and bc.indegree(7) == 1 and list(bc.adjacent(5)) == [(1, 2.0)]
    assert bigraph_continuous.from_packable(unpack(pack(bc))).e() == 2


def test_bigraph_continuous_from_file(tmp_path):
    f = _write(tmp_path, "bc.txt", ["3", "0,1,0.5", "2,0,1.5"])
    g = bigraph_continuous(f)
    out = []
    g.traverse(lambda a, b, c: out.append((a, b, c)))
    assert g.v() == 3 and out == [(0, 1, 0.5), (2, 0, 1.5)]
