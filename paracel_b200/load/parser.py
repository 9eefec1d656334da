"""Line parsers (reference: include/load/parser.hpp:33-116)."""
from __future__ import annotations

from functools import partial
from typing import Callable, List

from ..utils.ext import str_split


def parser_a_int(line: str, sep: str = " ") -> List[int]:
    return [int(x) for x in str_split(line, sep)]


def parser_a(line: str, sep: str = " ") -> List[str]:
    """``a b c d`` -> ['a', 'b', 'c', 'd']."""
    return str_split(line, sep)


def parser_b(line: str, sep1: str = " ", sep2: str = " ") -> List[str]:
    """``a b|c|d`` with (sep1=' ', sep2='|') -> ['a', 'b', 'c', 'd']."""
    tmp = str_split(line, sep1)
    return [tmp[0]] + str_split(tmp[1], sep2)


def gen_parser(parser: Callable, *seps: str) -> Callable[[str], List[str]]:
    """Bind the separators of a parser (1 to 3 argument forms of the reference)."""
    p = partial(parser, *[]) if not seps else (lambda line: parser(line, *seps))
    # remember what was bound so that the loader can use its native fast path
    try:
        p.pcl_base = parser
        p.pcl_seps = seps
    except AttributeError:  # pragma: no cover
        pass
    return p
