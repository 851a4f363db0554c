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


@pytest.mark.skipif(shutil.which("gcc") is None, reason="needs gcc")
def test_a_plain_c_host_links_and_gets_status_codes(tmp_path):
    """What INTEGRATION.md describes for a C host: include the header, link libcc1d.so, fill a block, call.
    No GPU is touched: argument validation comes before any launch."""
    libdir = os.path.join(ROOT, "causal_conv1d_b200")
    if not os.path.exists(os.path.join(libdir, "libcc1d.so")):
        pytest.skip("libcc1d.so not built")
    src = tmp_path / "host.c"
    src.write_text(r'''
#include <stdio.h>
#include <string.h>
#include "cc1d.h"
int main(void) {
    cc1d_fwd_params p;
    memset(&p, 0, sizeof p);
    p.itype = CC1D_BF16; p.wtype = CC1D_BF16; p.width = 9; p.silu = 1;
    p.batch = 1; p.dim = 8; p.seqlen = 16;
    p.x = (void *)0x1000; p.out = (void *)0x2000; p.weight = (void *)0x3000;
    p.x_batch_stride = 128; p.x_c_stride = 16; p.x_l_stride = 1;
    p.out_batch_stride = 128; p.out_c_stride = 16; p.out_l_stride = 1;
    p.weight_c_stride = 9; p.weight_width_stride = 1;
    int rc = cc1d_fwd(&p, (cc1d_stream_t)0);
    printf("%d %d %s\n", cc1d_abi_version(), rc, cc1d_status_str(rc));
    return rc == CC1D_ERR_WIDTH ? 0 : 1;
}
''')
    exe = tmp_path / "host"
    subprocess.run(["gcc", "-std=c99", "-Wall", "-Werror", "-I", os.path.join(ROOT, "include"), str(src), "-o", str(exe),
                    "-L", libdir, "-l:libcc1d.so", f"-Wl,-rpath,{libdir}"], check=True)
    out = subprocess.run([str(exe)], check=True, capture_output=True, text=True).stdout.split(None, 2)
    assert int(out[0]) >= 4 and "width" in out[2]
