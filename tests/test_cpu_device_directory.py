"""Key directory, handler registry and key filters of the device backend: the parts that need
no GPU (string keys <-> table rows, handler names, filter names)."""
from types import SimpleNamespace

import numpy as np
import pytest

from paracel_b200.ps.device_handlers import (is_device_handler, key_filter, register_device_handler,
                                             resolve_device_handler)
from paracel_b200.ps.device_store import TableEntry


def _entry(kind, rows, **kw):
    return TableEntry(kind, SimpleNamespace(rows=rows, width=4, device="cpu"), **kw)


def test_prefix_and_suffix_keys_map_to_rows():
    w = _entry("rows", 100, prefix="W_")
    pr = _entry("scalars", 50, suffix="_pr")
    bare = _entry("rows", 10)
    assert w.row_of("W_7") == 7 and w.key_of(7) == "W_7"
    assert w.row_of("W_100") is None          # outside the table
    assert w.row_of("H_7") is None and w.row_of("W_x") is None and w.row_of("W_") is None
    assert pr.row_of("49_pr") == 49 and pr.key_of(3) == "3_pr"
    assert pr.row_of("49_links") is None
    assert bare.row_of("9") == 9 and bare.row_of("10") is None and bare.row_of("theta") is None


def test_names_translate_original_ids():
    names = np.array([5, 17, 4000000000, 4000000007], dtype=np.int64)
    e = _entry("rows", 4, prefix="usr_bias_", names=names)
    assert e.row_of("usr_bias_17") == 1
    assert e.row_of("usr_bias_4000000007") == 3
    assert e.row_of("usr_bias_6") is None
    assert e.key_of(2) == "usr_bias_4000000000"


def test_dense_entries_match_their_exact_key_only():
    e = _entry("dense", 1, key="theta")
    assert e.row_of("theta") == 0 and e.row_of("theta_1") is None and e.pattern == "theta"


def test_reference_handler_names_resolve_to_kinds():
    for name in ("lr_theta_update", "mf_fac_updater", "mf_bias_updater", "cnt_updater", "svd_updater",
                 "default_incr_ld", "local_update_kmeans_clusters", "gLDA_word_update"):
        assert resolve_device_handler(name).kind == "add"
    assert resolve_device_handler("max_updater").kind == "max"
    assert not is_device_handler("no_such_handler")
    with pytest.raises(KeyError):
        resolve_device_handler("no_such_handler")
    register_device_handler("half_step", "sgd", lr=0.5)
    h = resolve_device_handler("half_step")
    assert h.kind == "sgd" and h.lr == 0.5
    with pytest.raises(ValueError):
        register_device_handler("bad", "multiply")


def test_key_filters_by_name_and_by_form():
    assert key_filter("", "mf_W_filter")("W_12") and not key_filter("", "mf_W_filter")("H_12")
    assert key_filter("", "pr_filter")("12_pr") and not key_filter("", "pr_filter")("12_links")
    assert key_filter("", "prefix:usr_")("usr_bias_1")
    assert key_filter("", "suffix:_cnt")("3_u_cnt")
    assert key_filter("", "contains:bias")("item_bias_9")
    assert key_filter("", "")("anything")


def test_graph_traverse_by_vertex_hands_out_vertex_and_neighbours():
    from paracel_b200.graph import digraph
    g = digraph()
    g.add_edge(1, 2, 0.5)
    g.add_edge(1, 3, 1.5)
    g.add_edge(2, 3, 2.5)
    seen = {}
    g.traverse_by_vertex(lambda item: seen.__setitem__(item[0], dict(item[1])))
    assert seen[1] == {2: 0.5, 3: 1.5} and seen[2] == {3: 2.5}
