"""The C header compiles as plain C, and the ctypes mirror used by the C-ABI tests has every
field of every parameter block at the offset the C compiler gives it (field names included: a
name that is not in the header does not compile)."""
import ctypes
import os
import shutil
import subprocess

import pytest

import cabi

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

BLOCKS = {
    "cc1d_fwd_params": cabi.FwdParams,
    "cc1d_bwd_params": cabi.BwdParams,
    "cc1d_peer_group": cabi.PeerGroup,
    "cc1d_update_params": cabi.UpdateParams,
    "cc1d_varlen_states_params": cabi.VarlenParams,
    "cc1d_prefill_varlen_params": cabi.PrefillParams,
}
if hasattr(cabi, "PeerAllreduceParams"):
    BLOCKS["cc1d_peer_allreduce_params"] = cabi.PeerAllreduceParams


@pytest.mark.skipif(shutil.which("gcc") is None, reason="needs gcc")
def test_header_is_plain_c_and_matches_the_ctypes_mirror(tmp_path):
    lines = ['#include <stdio.h>', '#include "cc1d.h"', "int main(void) {"]
    for cname, st in BLOCKS.items():
        lines.append(f'    printf("{cname} %zu\\n", sizeof({cname}));')
        for fname, _ in st._fields_:
            lines.append(f'    printf("{cname}.{fname} %zu\\n", offsetof({cname}, {fname}));')
    lines += ["    return 0;", "}"]
    src = tmp_path / "layout.c"
    src.write_text("\n".join(lines) + "\n")
    exe = tmp_path / "layout"
    subprocess.run(["gcc", "-std=c99", "-Wall", "-Werror", "-pedantic", "-I", os.path.join(ROOT, "include"),
                    str(src), "-o", str(exe)], check=True)
    got = dict(line.split() for line in subprocess.run([str(exe)], check=True, capture_output=True, text=True).stdout.splitlines())
    for cname, st in BLOCKS.items():
        assert int(got[cname]) == ctypes.sizeof(st), cname
        for fname, _ in st._fields_:
            assert int(got[f"{cname}.{fname}"]) == getattr(st, fname).offset, f"{cname}.{fname}"
