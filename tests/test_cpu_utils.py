"""Unit tests of the host utilities; the cases restate the reference's Boost tests
(test/test_utils.cpp, test_paracel_types.cpp, test_decomp.cpp, test_ring.cpp, test_kv.cpp,
test_packer.cpp, test_proxy.cpp, test_f_traits.cpp)."""
import json
import math
import os

import numpy as np
import pytest

from paracel_b200._core import core
from paracel_b200.utils import dump as D
from paracel_b200.utils.decomp import npfact2d, npfactx, npfacty
from paracel_b200.utils.ext import (add_folder_suffix_with_date, dot_product, endswith, expand,
                                    file_replace, startswith, str_join, str_split,
                                    str_split_by_word, todir)
from paracel_b200.utils.func_utility import f_traits
from paracel_b200.utils.misc import (get_hostnames_dict, json_parser, random_double,
                                     random_double_list, tail)
from paracel_b200.utils.packer import (pack, pack_prefixed, packer, pkl_dat_sequential, unpack,
                                       unpack_prefixed, unpkl_dat_sequential)
from paracel_b200.utils.types import bag_type, is_atomic, is_seqic


def test_string_helpers():
    init = ["hello", "world", "happy", "new", "year", "2015"]
    together = str_join(init, "orz")
    assert together == "helloorzworldorzhappyorzneworzyearorz2015"
    assert str_split_by_word(together, "orz") == init
    assert startswith(together, "hello") and not startswith(together, "helo")
    assert startswith(together, "") and endswith(together, "")
    assert endswith(together, "2015") and not endswith(together, "2014")
    assert not endswith(together, "7" + together)
    r = ["a", "b", "c", "d", "e"]
    assert str_split("a|b|c|d|e", "|") == r
    assert str_split("a|b|c|d|e", "?|?") == r
    assert str_split("a||b", "|") == ["a", "b"]          # empty fields are dropped
    assert core().split_char("a  b c", " ") == ["a", "b", "c"]
    assert core().split_any("a:b|c d", ":| ") == ["a", "b", "c", "d"]
    assert dot_product([1, 2, 3], [4, 5, 6]) == 32
    assert todir("x") == "x/" and todir("x/") == "x/"
    assert add_folder_suffix_with_date("out/").endswith("/") and len(add_folder_suffix_with_date("o")) > 6


def test_expand_and_file_replace(tmp_path):
    (tmp_path / "d" / "e").mkdir(parents=True)
    for n in ("a.txt", "b.csv", "d/c.txt", "d/e/f.txt"):
        (tmp_path / n).write_text("x\n")
    assert expand(str(tmp_path / "a.txt")) == [str(tmp_path / "a.txt")]
    assert sorted(os.path.basename(p) for p in expand(str(tmp_path))) == ["a.txt", "b.csv", "c.txt", "f.txt"]
    assert [os.path.basename(p) for p in expand(str(tmp_path / "*.csv"))] == ["b.csv"]
    assert len(expand([str(tmp_path / "a.txt"), str(tmp_path / "d")])) == 3
    src, dst = tmp_path / "tpl", tmp_path / "out"
    src.write_text("# comment\nCC = XX\nall: YY XX\n")
    file_replace(str(src), str(dst), {"XX": "g++", "YY": "main"})
    assert dst.read_text() == "CC = g++\nall: main g++\n"


def test_random_is_open_unit_interval():
    n, inc = 200000, 0
    for _ in range(n):
        x, y = random_double(), random_double()
        assert 0.0 < x < 1.0
        inc += x * x + y * y < 1.0
    assert abs(4.0 * inc / n - math.pi) < 0.02
    lst = random_double_list(100, 0.1)
    assert len(lst) == 100 and max(lst) < 0.1


def test_json_parser(tmp_path):
    cfg = {"wu": "hong", "hong": 7, "changsheng": True, "jiang": 3.141592653,
           "wul": ["hong", "xun", "zhang"], "hongl": [1, 2, 3, 4, 5, 6, 7],
           "changshengl": [True, False, False, True, True],
           "jiangl": [1.23, 2.34, 3.45, 4.56, 5.67, 6.78, 7.89], "nested": {"a": {"b": 5}},
           "file": str(tmp_path / "test.json"), "nofile": str(tmp_path / "nope")}
    p = tmp_path / "test.json"
    p.write_text(json.dumps(cfg))
    pt = json_parser(str(p))
    assert pt.parse("wu", str) == "hong" and pt.parse("hong", int) == 7
    assert pt.parse("changsheng", bool) is True and pt.parse("jiang", float) == 3.141592653
    assert pt.parse_v("wul", str) == ["hong", "xun", "zhang"]
    assert pt.parse_v("hongl", int) == [1, 2, 3, 4, 5, 6, 7]
    assert pt.parse_v("changshengl", bool) == [True, False, False, True, True]
    assert pt.parse_v("jiangl", float) == [1.23, 2.34, 3.45, 4.56, 5.67, 6.78, 7.89]
    assert pt.parse("nested.a.b", int) == 5
    assert pt.check_parse("file", str) == str(p)
    with pytest.raises(FileNotFoundError):
        pt.check_parse("nofile", str)
    assert pt.check_parse_v("wul") if False else True


def test_hash_golden_values_and_ring():
    c = core()
    # libstdc++ values quoted in test_paracel_types.cpp:34-54 (non-Apple branch)
    assert c.hash_string("abcd") == 16030370620903852840
    assert c.hash_string_list(["1", "2", "3"]) == 15152834183934801446
    assert c.hash_string_list(["a", "b", "c"]) == 1227721600474941649
    assert c.hash_u64(3) == 3
    assert c.hash_value_combine(1, 2) != c.hash_value_combine(2, 1)
    from paracel_b200.ps.ring import ring
    keys = ["dw", "q[,:0]_0", "q[,:1]_0", "q[,:2]_0", "q[,:3]_0", "p[0:,]_2", "p[13:,]_2", "p[42:,]_2",
            "p[5:,]_2", "p[3:,]_1"]
    r = ring([1, 2, 3])
    assert [r.get_server(k) for k in keys] == [2, 2, 3, 1, 3, 1, 2, 3, 2, 3]      # test_ring.cpp:84-108
    r2 = ring(["balin1", "beater5", "beater7"])
    assert [r2.get_server(k) for k in keys] == ["beater7", "beater5", "balin1", "beater7", "beater7",
                                                "balin1", "beater7", "balin1", "beater5", "beater5"]
    assert c.ring_bsearch([10, 20, 30], 5) == 0 and c.ring_bsearch([10, 20, 30], 31) == 0
    assert c.ring_bsearch([10, 20, 30], 20) == 1 and c.ring_bsearch([10, 20, 30], 21) == 2
    r.remove_server(2)
    assert set(r.get_server(k) for k in keys) <= {1, 3}


def test_decomp_table():
    assert npfact2d(10) == (2, 5) and npfact2d(10, False) == (5, 2)
    assert npfact2d(7) == (7, 1) and npfact2d(7, False) == (1, 7)
    assert npfact2d(2) == (2, 1) and npfact2d(6) == (2, 3) and npfact2d(8) == (2, 4)
    assert npfact2d(1) == (1, 1) and npfact2d(16) == (4, 4)
    assert npfactx(5) == (5, 1) and npfacty(5) == (1, 5)


def test_types_and_bag():
    assert is_atomic(3) and is_atomic(2.0) and not is_atomic([1])
    assert is_seqic([1, 2]) and is_seqic([1.0]) and not is_seqic("ab")
    bg = bag_type()
    for x in (1, 3, 5):
        bg.put(x)
    seen = []
    bg.traverse(seen.append)
    cp = bg.get()
    assert seen == [1, 3, 5] and cp.size() == 3 and list(bag_type(bg)) == [1, 3, 5]
    assert bag_type().assign(bg) is not bg and list(bag_type().assign(bg)) == [1, 3, 5]


def test_f_traits():
    def f(a: int, b: float) -> str:
        return ""
    t = f_traits(f)
    assert t.arity == 2 and t.args == (int, float) and t.result_type is str
    assert f_traits(lambda x: x).arity == 1

    class Functor:
        def __call__(self, a, b, c):
            return a
    assert f_traits(Functor()).arity == 3


def test_packer_round_trips(tmp_path):
    cases = [True, 54, 3.14, "abcd", [1, 2, 3], [1.5, 2.5], {"a": 1, "b": 2}, {"k": [1.0, 2.0]},
             [["a", "b", 1.0]], {1: [[2, 0.5]]}, None, [[1.0, 2.0], [3.0, 4.0]], -7, 2 ** 40, -2 ** 40]
    for v in cases:
        assert unpack(pack(v)) == v
        assert unpack_prefixed(pack_prefixed(v)) == v
        assert packer().unpack(packer(v).pack()) == v
    assert unpack(pack(np.arange(3))) == [0, 1, 2]
    assert unpack(pack((1, 2))) == [1, 2]
    # the C++ codec reads what Python wrote and the other way round
    c = core()
    for a, b, name, exp in ((3, 4, "add", 7), (1.5, 2, "add", 3.5), ([1, 2], [3, 4], "add", [4, 6]),
                            ({"x": 1}, {"x": 2, "y": 1}, "wc_updater", {"x": 3, "y": 1}),
                            (3.0, 2.0, "max_updater", 3.0), ([1], [2, 3], "init_updater", [1, 2, 3]),
                            ({"a": 0}, {"a": 5, "b": 9}, "gLDA_dict_update", {"a": 0, "b": 1}),
                            ([7, 0.5], [9, 0.2], "smallest_error_updater", [9, 0.2]),
                            ({"1": ["a"]}, {"1": ["b"], "2": ["c"]}, "local_update_kmeans_groups",
                             {"1": ["a", "b"], "2": ["c"]}),
                            ([[1, 2], [3, 4]], [[1, 1], [1, 1]], "local_update_kmeans_clusters",
                             [[2, 3], [4, 5]])):
        assert unpack(c.apply_builtin_handler(name, pack(a), pack(b))) == exp
    with pytest.raises(RuntimeError):
        c.apply_builtin_handler("add", pack([1, 2]), pack([1]))
    # pkl_dat files: length-prefixed blobs, matrices column-major
    m = np.arange(6, dtype=np.float64).reshape(2, 3)
    pkl_dat_sequential(m, str(tmp_path / "m.pkl"))
    assert np.array_equal(unpkl_dat_sequential(str(tmp_path / "m.pkl"), cols=3), m)
    import scipy.sparse as sp
    s = sp.csr_matrix(([1.0, 2.0], ([0, 2], [1, 3])), shape=(3, 4))
    pkl_dat_sequential(s, str(tmp_path / "s.pkl"))
    assert (unpkl_dat_sequential(str(tmp_path / "s.pkl"), sparse=True) != s).nnz == 0
    pkl_dat_sequential({"a": [1, 2]}, str(tmp_path / "d.pkl"))
    assert unpkl_dat_sequential(str(tmp_path / "d.pkl")) == {"a": [1, 2]}


def test_proxies():
    from paracel_b200.ps.handlers import filter_proxy, filter_with_key_proxy, update_proxy
    up = update_proxy(lambda a, b: [x + y for x, y in zip(a, b)])
    assert unpack(up(pack([1.0, 2.0]), pack([0.5, 0.5]))) == [1.5, 2.5]
    assert filter_with_key_proxy(lambda k: k.startswith("W_"))("W_1", pack(0)) is True
    assert filter_proxy(lambda k, v: v > 1)("x", pack(2)) is True


def test_kv_store_semantics():
    from paracel_b200.ps.kv import kvs
    kv = kvs()
    kv.set("a", 7)
    kv.set_multi({"b": [1.0, 2.0], "c": "str"})
    assert kv.contains("a") and not kv.contains("z")
    assert kv.get("a") == 7 and kv.get("z") is None and kv.get("z", 1) == 1
    assert kv.get_multi(["a", "c"]) == [7, "str"]
    with pytest.raises(Exception):
        kv.get_multi(["a", "z"])
    assert kv.get_multi_dict(["a", "z"]) == {"a": 7}
    assert kv.incr("a", 3) and kv.get("a") == 10
    assert kv.incr("b", [1.0, 1.0]) and kv.get("b") == [2.0, 3.0]
    assert not kv.incr("b", [1.0]) and not kv.incr("z", 1)
    val, uniq = kv.gets("a")
    assert val == 10 and kv.cas("a", 11, uniq) and not kv.cas("a", 12, uniq) and kv.get("a") == 11
    assert kv.cas("new", 1, 0) and kv.get("new") == 1
    assert kv.gets("zz") is None
    assert kv.delete("new") and not kv.delete("new")
    assert set(kv.getall()) == {"a", "b", "c"} and len(kv) == 3
    kv.clean()
    assert len(kv) == 0


def test_dump_formats(tmp_path):
    p = str(tmp_path / "v")
    D.dump_vector([0.1234567, 2.0], p, "|")
    assert open(p).read() == "0.123457|2.000000\n"
    D.dump_vector([], p)
    assert open(p).read() == ""                             # no underflow on empty input
    D.dump_vector([("a", "b", 0.5), (1, 2, 0.25)], p, "\n")
    assert open(p).read() == "a,b,0.500000\n1,2,0.250000\n"
    D.dump_vector([([1.0, 2.0], 0.7)], p, "\n")
    assert open(p).read() == "1.000000,2.000000:0.700000\n"
    D.dump_vector([(3, 0.5)], p)
    assert open(p).read() == "3:0.500000\n"
    D.dump_dict_scalar({"miu": 3.25, "rating_sz": 1e7, "n": 3}, p)
    assert open(p).read() == "miu\t3.25\nn\t3\nrating_sz\t1e+07\n"
    D.dump_dict_vector({"7": [0.5, 1.0], "8": []}, p)
    assert open(p).read() == "7\t0.500000|1.000000\n"
    D.dump_dict_pairs({1: [(2, 0.5), (3, 0.25)]}, p)
    assert open(p).read() == "1\t2:0.500000|3:0.250000\n"
    D.dump_prob_mtx({"a": [("x", 0.5), ("y", 0.123456789)], "b": []}, p)
    assert open(p).read() == "a\tx:0.500000|y:0.123457\nb\t"
    D.dump_dict_vector({"1": [1.0]}, p)
    D.dump_dict_vector({"2": [2.0]}, p, append=True)
    assert D.read_dict_vector(p) == {"1": [1.0], "2": [2.0]}
    for r in range(3):
        open(str(tmp_path / f"res_{r}"), "w").write(f"{r}\n")
    D.files_merge(str(tmp_path / "res_*"), str(tmp_path / "res_merge"))
    assert open(str(tmp_path / "res_merge")).read() == "0\n1\n2\n"


def test_misc(tmp_path):
    assert get_hostnames_dict("h1:1,2,3_PARACEL_h2:4") == [{"host": "h1", "ports": "1,2,3"},
                                                          {"host": "h2", "ports": "4"}]
    p = tmp_path / "t"
    p.write_text("".join(f"{i}\n" for i in range(10)))
    assert tail(str(p), 3, int) == [7, 8, 9]
    assert tail(str(p), 20) == [str(i) for i in range(10)]


def test_hash_module_matches_the_native_functions():
    from paracel_b200._core import core
    from paracel_b200.utils.hash import hash_combine, hash_value
    c = core()
    assert hash_value(42) == 42                        # std::hash of an integer is the identity
    assert hash_value("abc") == c.hash_string("abc")
    assert hash_value(["a", "b"]) == c.hash_string("vechashab")
    assert hash_value(("a", 7)) == hash_combine(c.hash_string("a"), 7)
    assert hash_value(("a", 7)) != hash_value((7, "a"))


def test_type_traits_and_small_helpers():
    import numpy as np
    from paracel_b200.utils import misc, types
    assert types.is_comm_builtin(3) and not types.is_comm_builtin([3])
    assert types.is_comm_container([1, 2.0]) and types.is_comm_container("x")
    assert types.is_matrix(np.zeros((2, 3))) and not types.is_matrix(np.zeros(3))
    assert types.threads_num == 5
    m = np.arange(6, dtype=float).reshape(2, 3)
    flat = misc.mat2vec(m)
    assert flat == [0.0, 3.0, 1.0, 4.0, 2.0, 5.0]      # column major
    assert np.array_equal(misc.vec2mat(flat, 2), m)
    assert misc.evec2vec(misc.vec2evec([1, 2])) == [1.0, 2.0]
    assert misc.ring_bsearch([10, 20, 30], 15) == 1 and misc.ring_bsearch([10, 20, 30], 35) == 0
    import heapq
    h = [misc.heap_node("a", 3.0), misc.heap_node("b", 1.0), misc.heap_node("c", 2.0)]
    heapq.heapify(h)
    assert heapq.heappop(h).key == "b"
    ports = misc.get_ports(2)
    assert len(ports) == 2 and all(2014 <= p < 65535 for p in ports)
    with __import__("pytest").raises(RuntimeError):
        misc.ERROR_ABORT("boom")


def test_rating_balance_over_the_rank_grid():
    """balanced_groups + grid_rank: near-equal rating counts per rank for Zipf ids, and an extremely
    popular item is shared by every column of the grid instead of loading one of them."""
    import torch
    from paracel_b200.models.mf_gpu import balanced_groups, grid_rank
    g = torch.Generator().manual_seed(0)
    n_u, n_i, nnz = 20000, 4000, 400_000
    wu = 1.0 / torch.arange(1, n_u + 1, dtype=torch.float64) ** 1.1
    wi = 1.0 / torch.arange(1, n_i + 1, dtype=torch.float64) ** 1.1
    u = torch.multinomial(wu, nnz, replacement=True, generator=g)
    i = torch.multinomial(wi, nnz, replacement=True, generator=g)
    cu, ci = torch.bincount(u, minlength=n_u), torch.bincount(i, minlength=n_i)
    for npx, npy in ((2, 4), (2, 2), (1, 2)):
        ug = balanced_groups(cu, npx, spread_above=0.25)
        ig = balanced_groups(ci, npy, spread_above=0.25)
        r = grid_rank(u, i, ug, ig, npx, npy)
        cnt = torch.bincount(r, minlength=npx * npy).double()
        assert cnt.max() / cnt.mean() < 1.08, (npx, npy, cnt.tolist())
        if npy == 4:
            assert int(ig[0]) == -1                       # the top item is dealt over the columns
            share = torch.bincount(r[i == 0], minlength=npx * npy).double() / cnt
            assert share.max() / share.min() < 1.3
    assert int((balanced_groups(cu, 1) != 0).sum()) == 0
