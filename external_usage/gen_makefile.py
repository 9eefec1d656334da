#!/usr/bin/env python
"""Writes ``Makefile`` next to this script with the include directory of the installed
paracel_b200 filled in (the reference's external_usage generator does the same with
``file_replace`` and its install prefix)."""
import os

import paracel_b200
from paracel_b200.utils.ext import file_replace

here = os.path.dirname(os.path.abspath(__file__))
inc = os.path.join(os.path.dirname(os.path.abspath(paracel_b200.__file__)), "csrc", "core")
file_replace(os.path.join(here, "Makefile.template"), os.path.join(here, "Makefile"),
             {"PARACEL_INCLUDE_DIR": inc})
print("wrote", os.path.join(here, "Makefile"))
