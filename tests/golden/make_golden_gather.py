"""Golden fixtures for the decode update with ``conv_state_indices`` (a pool of states, gathered
per batch entry; negative index = padded entry), from the REFERENCE's own PyTorch function.

    python tests/golden/make_golden_gather.py <reference checkout>

``causal_conv1d_update_ref`` (``causal_conv1d/causal_conv1d_interface.py:205-242``) has no
``conv_state_indices`` argument; the reference pins the gathered path the way its own test does
(``tests/test_causal_conv1d.py:199-233``, ``:250-321``): the rows named by the non-negative
indices are gathered, ``causal_conv1d_update_ref`` runs on them, and the updated rows are
scattered back; a padded entry outputs exactly zero and its (non-existent) row, like every row
that no index names, is left untouched (``csrc/causal_conv1d_update.cu:43-54``).  Written to
``golden_gather.npz`` / ``golden_gather.json``.  Nothing here is imported by the product.
"""
import json
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, HERE)
from make_golden import DT, f32, load_reference  # noqa: E402


def main(ref_path):
    _, update_ref, _ = load_reference(ref_path)
    arrays, meta = {}, {}
    k = 0
    for width in (2, 3, 4):
        for seqlen in (1, 4):
            for circ in (False, True):
                for itype, wtype in (("fp32", "fp32"), ("bf16", "fp32"), ("fp16", "fp16")):
                    k += 1
                    if k % 2 == 0:
                        continue
                    torch.manual_seed(500 + k)
                    batch, entries, dim = 6, 11, 16
                    state_len = (8 if circ else width - 1 + (k % 3))
                    x = torch.randn(batch, dim, seqlen).to(DT[itype])
                    pool = torch.randn(entries, dim, state_len).to(DT[itype])
                    weight = torch.randn(dim, width).to(DT[wtype])
                    bias = torch.randn(dim).to(DT[wtype]) if k % 3 else None
                    idx = torch.randperm(entries)[:batch].int()
                    if k % 4 != 1:
                        idx[k % batch] = -1
                        idx[(k + 3) % batch] = -1
                    cache = torch.randint(0, 1024, (batch,), dtype=torch.int32) if circ else None
                    silu = k % 5 != 0
                    valid = idx >= 0
                    rows = pool[idx[valid].long()].clone()
                    out_valid = update_ref(x[valid], rows, weight, bias, activation="silu" if silu else None,
                                           cache_seqlens=None if cache is None else cache[valid])
                    out = torch.zeros(batch, dim, seqlen, dtype=DT[itype])
                    out[valid] = out_valid
                    pool_out = pool.clone()
                    pool_out[idx[valid].long()] = rows
                    name = f"ga_w{width}_l{seqlen}_c{int(circ)}_{itype}_{wtype}"
                    for key, v in dict(x=f32(x), conv_state=f32(pool), weight=f32(weight), bias=f32(bias),
                                       conv_state_indices=idx.numpy(), out=f32(out), conv_state_out=f32(pool_out),
                                       cache_seqlens=None if cache is None else cache.numpy()).items():
                        if v is not None:
                            arrays[f"{name}/{key}"] = v
                    meta[name] = dict(kind="update_gather", itype=itype, wtype=wtype, width=width, silu=silu,
                                      has_bias=bias is not None, circular=circ, padded=bool((idx < 0).any()))
    np.savez_compressed(os.path.join(HERE, "golden_gather.npz"), **arrays)
    with open(os.path.join(HERE, "golden_gather.json"), "w") as f:
        json.dump({"torch": torch.__version__, "cases": meta}, f, indent=1, sort_keys=True)
    print(f"{len(meta)} cases, {sum(a.nbytes for a in arrays.values()) / 1e3:.1f} KB raw")


if __name__ == "__main__":
    if len(sys.argv) != 2:
        raise SystemExit(__doc__)
    main(sys.argv[1])
