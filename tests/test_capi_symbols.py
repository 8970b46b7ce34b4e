"""The C-ABI library loads without a GPU and exports every function include/ge2_b200.h declares."""
import ctypes
import re
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parents[1]


def declared_functions():
    text = (ROOT / "include" / "ge2_b200.h").read_text()
    return sorted(set(re.findall(r"GE2_API[^;(]*?\b(ge2_\w+)\s*\(", text)))


def test_header_declares_functions():
    names = declared_functions()
    assert "ge2_unique_bitmap" in names and "ge2_lp_step" in names and "ge2_adagrad_scatter" in names
    assert len(names) >= 17


def test_library_exports_every_declared_symbol(ge2):
    lib = ge2.load_library()
    for name in declared_functions():
        assert hasattr(lib, name), f"{name} declared in include/ge2_b200.h but not exported"
    assert sorted(ge2.capi.EXPORTS) == [n for n in declared_functions() if n in ge2.capi.EXPORTS]
    assert set(declared_functions()) <= set(ge2.capi.EXPORTS)


def test_host_only_entry_points(ge2):
    lib = ge2.load_library()
    assert lib.ge2_version().startswith(b"ge2_b200")
    assert lib.ge2_status_string(0) == b"ok"
    assert lib.ge2_unique_workspace_bytes(0) == 0
    assert lib.ge2_unique_workspace_bytes(1_000_000) >= 125_000 + 62_500
    # argument validation happens before any CUDA call
    assert lib.ge2_unique_bitmap(None, -1, 10, None, 0, None, None, None, None) == 1
    d = ge2.capi.LpDesc()
    out = ctypes.c_size_t(0)
    assert lib.ge2_lp_workspace_bytes(ctypes.byref(d), ctypes.byref(out)) == 1


def test_desc_struct_matches_header_size(ge2):
    """ctypes mirror and C struct agree in size (a C probe compiled against the header prints sizeof)."""
    import subprocess
    import tempfile

    src = '#include "ge2_b200.h"\n#include <stdio.h>\nint main(){printf("%zu %zu %zu", sizeof(ge2_lp_desc), offsetof(ge2_lp_desc, workspace), offsetof(ge2_lp_desc, rel));return 0;}'
    with tempfile.TemporaryDirectory() as td:
        c = Path(td) / "p.c"
        c.write_text(src)
        exe = Path(td) / "p"
        r = subprocess.run(["gcc", "-I", str(ROOT / "include"), str(c), "-o", str(exe)], capture_output=True, text=True)
        if r.returncode != 0:
            pytest.skip("no C compiler: " + r.stderr[:80])
        size, off_ws, off_rel = map(int, subprocess.run([str(exe)], capture_output=True, text=True).stdout.split())
    D = ge2.capi.LpDesc
    assert ctypes.sizeof(D) == size and D.workspace.offset == off_ws and D.rel.offset == off_rel


def test_swap_and_eval_structs_match_header(ge2):
    """the ctypes mirrors of ge2_swap_desc and ge2_eval_desc agree with the C structs in size and in the offsets of a few members"""
    import subprocess
    import tempfile

    src = ('#include "ge2_b200.h"\n#include <stdio.h>\n#include <stddef.h>\nint main(){printf("%zu %zu %zu %zu %zu %zu", sizeof(ge2_swap_desc), '
           'offsetof(ge2_swap_desc, slab_bytes), offsetof(ge2_swap_desc, status), sizeof(ge2_eval_desc), offsetof(ge2_eval_desc, neg_ids), '
           'offsetof(ge2_eval_desc, workspace));return 0;}')
    with tempfile.TemporaryDirectory() as td:
        c = Path(td) / "p.c"
        c.write_text(src)
        exe = Path(td) / "p"
        r = subprocess.run(["gcc", "-std=c99", "-I", str(ROOT / "include"), str(c), "-o", str(exe)], capture_output=True, text=True)
        if r.returncode != 0:
            pytest.skip("no C compiler: " + r.stderr[:80])
        s_size, s_slab, s_status, e_size, e_neg, e_ws = map(int, subprocess.run([str(exe)], capture_output=True, text=True).stdout.split())
    S, E = ge2.capi.SwapDesc, ge2.capi.EvalDesc
    assert ctypes.sizeof(S) == s_size and S.slab_bytes.offset == s_slab and S.status.offset == s_status
    assert ctypes.sizeof(E) == e_size and E.neg_ids.offset == e_neg and E.workspace.offset == e_ws
