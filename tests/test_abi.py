"""The C-ABI library without a GPU: it loads, exports every symbol the header declares, reports
errors through the error-string convention and refuses to work without a CUDA device."""
import ctypes as C
import os
import re

import numpy as np
import pytest

from cuml_b200.fil import _lib
from cuml_b200.fil._desc import CCreateOpts, CInfo
from tests.conftest import ROOT, has_gpu
from tests.helpers import random_forest_desc


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "b2fil.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(b2fil_[a-z_0-9]+)\s*\(", text)))


def test_header_symbols_are_exported(lib):
    names = declared_symbols()
    assert "b2fil_predict" in names and "b2fil_forest_create" in names and len(names) >= 12
    for n in names:
        assert hasattr(lib, n), f"{n} is declared in include/b2fil.h but not exported"


def test_version_and_error_string(lib):
    assert lib.b2fil_version() >= 100
    rc = lib.b2fil_forest_create(None, None, None)
    assert rc == -1
    assert b"NULL" in lib.b2fil_last_error()
    assert lib.b2fil_forest_free(None) == 0
    info = CInfo()
    assert lib.b2fil_forest_info(None, C.byref(info)) == -1
    assert lib.b2fil_output_elems_per_row(None, 0) == 0
    assert lib.b2fil_predict(None, 0, None, 0, 0, None, 0, 0.5, None) == -1


def test_struct_sizes_match_header():
    # the header's structs, compiled by gcc, must have the sizes of the ctypes mirrors
    import subprocess
    import tempfile

    from cuml_b200.fil._desc import CForestDesc

    src = ('#include <stdio.h>\n#include "b2fil.h"\nint main(){printf("%zu %zu %zu\\n", '
           "sizeof(b2fil_forest_desc), sizeof(b2fil_create_opts), sizeof(b2fil_info));return 0;}")
    with tempfile.TemporaryDirectory() as d:
        c = os.path.join(d, "s.c")
        open(c, "w").write(src)
        exe = os.path.join(d, "s")
        subprocess.check_call(["gcc", "-I", os.path.join(ROOT, "include"), c, "-o", exe])
        sizes = [int(x) for x in subprocess.check_output([exe]).split()]
    assert sizes == [C.sizeof(CForestDesc), C.sizeof(CCreateOpts), C.sizeof(CInfo)]


@pytest.mark.skipif(has_gpu(), reason="checks the behaviour on a box without a GPU")
def test_no_gpu_means_error_not_fallback(lib):
    from cuml_b200.fil import ForestInference

    desc = random_forest_desc(0)
    with pytest.raises(_lib.B2FilError) as ei:
        ForestInference.load_from_treelite_model(desc)
    assert ei.value.code == -4


def test_python_argument_validation():
    from cuml_b200.fil import ForestInference

    with pytest.raises(ValueError):
        ForestInference(layout="zigzag")
    with pytest.raises(ValueError):
        ForestInference(precision="half")
    with pytest.raises(ValueError):
        ForestInference(default_chunk_size=3)
    with pytest.raises(ValueError):
        ForestInference(storage="ragged")


def test_product_never_imports_the_oracle():
    # the oracle is test infrastructure: nothing under cuml_b200/ may name it
    for dirpath, _, files in os.walk(os.path.join(ROOT, "cuml_b200")):
        for fn in files:
            if fn.endswith((".py", ".cu", ".cpp", ".hpp", ".h")):
                text = open(os.path.join(dirpath, fn)).read()
                assert "fil_oracle" not in text and "import oracle" not in text, fn
                assert "from oracle" not in text, fn
