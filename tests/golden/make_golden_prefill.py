"""Golden fixtures for the packed variable-length prefill with per-sequence conv states,
generated from the REFERENCE's own PyTorch functions.

    python tests/golden/make_golden_prefill.py <reference checkout>

The reference has no single call for this case; its semantics are pinned the way the
reference's seq_idx test pins its kernel (``tests/test_causal_conv1d.py:448-454``): the pack
is split and ``causal_conv1d_ref`` runs per sequence, here with ``initial_states`` taken from
a state pool and ``return_final_states=True``.  With ``state_len == width - 1`` the final
state is what ``causal_conv1d_ref`` returns; with a longer state and no prefix it is what
``causal_conv1d_varlen_states_ref`` returns; with both it is the last ``state_len`` entries
of ``[prefix | x_s]`` (the rule both functions share).  Writes ``golden_prefill.npz`` /
``golden_prefill.json``.  Nothing here is imported by the product.
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
    conv_ref, _, varlen_ref = load_reference(ref_path)
    arrays, meta = {}, {}
    k = 0
    for width in (2, 3, 4):
        for itype in ("fp32", "bf16", "fp16"):
            for extra in (0, 2):            # state_len = width - 1 + extra
                for mode in ("all", "mixed", "none"):
                    k += 1
                    torch.manual_seed(500 + k)
                    dim, S = 16, width - 1 + extra
                    lens = [5, 1, 2, 9, 3, 1, 12][: 4 + k % 4]
                    if k % 5 == 0:
                        lens[2] = 0              # an empty sequence keeps its state
                    pad = 3 if k % 2 else 0      # tokens after the last sequence
                    cu = np.concatenate([[0], np.cumsum(lens)]).astype(np.int32)
                    total = int(cu[-1]) + pad
                    nseq = len(lens)
                    x = torch.randn(total, dim).to(DT[itype])
                    weight = torch.randn(dim, width)
                    bias = torch.randn(dim) if k % 3 else None
                    silu = k % 4 != 0
                    rows = nseq + 3
                    pool = torch.randn(rows, dim, S).to(DT[itype])
                    idx = torch.randperm(rows)[:nseq].to(torch.int32)
                    has = {"all": torch.ones(nseq, dtype=torch.bool),
                           "none": torch.zeros(nseq, dtype=torch.bool),
                           "mixed": torch.arange(nseq) % 2 == 0}[mode]
                    out = torch.zeros(total, dim, dtype=DT[itype])
                    new_pool = pool.clone()
                    for s in range(nseq):
                        beg, end = int(cu[s]), int(cu[s + 1])
                        r = int(idx[s])
                        prefix = pool[r] if has[s] else torch.zeros(dim, S, dtype=DT[itype])
                        xs = x[beg:end].T.unsqueeze(0)
                        if end > beg:
                            ini = prefix[:, S - (width - 1):].unsqueeze(0) if has[s] else None
                            o, fs = conv_ref(xs, weight, bias, initial_states=ini, return_final_states=True,
                                             activation="silu" if silu else None)
                            out[beg:end] = o[0].T
                            if extra == 0:
                                new_pool[r] = fs[0]
                            elif not has[s]:
                                new_pool[r] = varlen_ref(x[beg:end], torch.tensor([0, end - beg]), S)[0]
                            else:
                                new_pool[r] = torch.cat([prefix, xs[0]], dim=1)[:, -S:]
                        else:
                            new_pool[r] = prefix
                    name = f"pf_w{width}_{itype}_s{S}_{mode}"
                    for key, v in dict(x=f32(x), weight=f32(weight), bias=f32(bias), cu_seqlens=cu,
                                       state_indices=idx.numpy(), has_initial_state=has.numpy(),
                                       conv_states=f32(pool), out=f32(out), conv_states_out=f32(new_pool)).items():
                        if v is not None:
                            arrays[f"{name}/{key}"] = v
                    meta[name] = dict(kind="prefill_varlen", itype=itype, width=width, silu=silu,
                                      has_bias=bias is not None, state_len=S, mode=mode)
    np.savez_compressed(os.path.join(HERE, "golden_prefill.npz"), **arrays)
    with open(os.path.join(HERE, "golden_prefill.json"), "w") as f:
        json.dump({"torch": torch.__version__, "cases": meta}, f, indent=1, sort_keys=True)
    print(f"{len(meta)} cases, {sum(a.nbytes for a in arrays.values()) / 1e6:.2f} MB raw")


if __name__ == "__main__":
    if len(sys.argv) != 2:
        raise SystemExit(__doc__)
    main(sys.argv[1])
