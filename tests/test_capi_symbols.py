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


def test_selected_negative_entry_points_validate_before_any_cuda_call(ge2):
    """Shapes the reference rejects with TORCH_CHECK (distmult_selected_neg_cuda.cpp:63-76, .cu:215-217) come back as
    GE2_ERR_INVALID_ARGUMENT; D above the kernels' 128 as GE2_ERR_UNSUPPORTED; empty inputs are accepted without a launch."""
    lib = ge2.load_library()
    p = 4096  # never dereferenced: every call below returns before it touches the device
    tour = lambda chunks, rows, negs, sel, D: lib.ge2_tournament_select(p, p, None, None, chunks, rows, negs, sel, D, p, p, None)  # noqa: E731
    assert tour(2, 5, 10, 3, 8) == 1       # negatives not divisible into groups
    assert tour(2, 5, 10, 0, 8) == 1
    assert tour(2, 5, 10, 5, 129) == 4     # D > 128
    assert tour(70000, 5, 10, 5, 8) == 4   # more chunks than a grid dimension holds
    assert tour(0, 5, 10, 5, 8) == 0 and tour(2, 0, 10, 5, 8) == 0
    fwd = lambda kind, chunks, rows, negs, sel, D: lib.ge2_selected_neg_scores(kind, p, p, p, chunks, rows, negs, sel, D, p, None, None)  # noqa: E731
    assert fwd(0, 1, 1, 1, 1, 8) == 1      # SelectedNegScoreKind::NONE
    assert fwd(3, 1, 1, 1, 1, 8) == 1
    assert fwd(1, 1, 1, 0, 1, 8) == 1      # no negatives to index
    assert fwd(2, 1, 1, 1, 1, 200) == 4
    assert fwd(1, 3, 0, 5, 2, 8) == 0 and fwd(2, 3, 4, 5, 0, 8) == 0
    assert lib.ge2_selected_neg_scores_backward(7, p, p, p, p, 1, 1, 1, 1, 8, p, p, None, None) == 1


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
