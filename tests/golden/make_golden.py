"""Generate the golden fixtures in this directory from the REFERENCE's own PyTorch functions.

Run once, in a container that has the reference checkout (it is not needed at test time):

    python tests/golden/make_golden.py <reference checkout>

The reference package is imported from the given path with its compiled module
``causal_conv1d_cuda`` stubbed (``causal_conv1d/cpp_functions.py:5`` imports it, the
pure-PyTorch functions never call it).  Outputs of ``causal_conv1d_ref``,
``causal_conv1d_update_ref`` and ``causal_conv1d_varlen_states_ref`` — and the gradients
autograd derives from them — are written with their inputs to ``golden.npz`` (float32 /
int arrays; 16-bit values are stored upcast, which is exact) plus ``golden.json`` (case
metadata).  Nothing here is imported by the product.
"""
import json
import os
import sys
import types

import numpy as np
import torch
import torch.nn.functional as F

HERE = os.path.dirname(os.path.abspath(__file__))
DT = {"fp32": torch.float32, "fp16": torch.float16, "bf16": torch.bfloat16}


def load_reference(path):
    sys.path.insert(0, path)
    sys.modules["causal_conv1d_cuda"] = types.ModuleType("causal_conv1d_cuda")
    from causal_conv1d.causal_conv1d_interface import causal_conv1d_ref, causal_conv1d_update_ref
    from causal_conv1d.causal_conv1d_varlen import causal_conv1d_varlen_states_ref
    return causal_conv1d_ref, causal_conv1d_update_ref, causal_conv1d_varlen_states_ref


def f32(t):
    return None if t is None else t.detach().float().cpu().numpy()


def main(ref_path):
    conv_ref, update_ref, varlen_ref = load_reference(ref_path)
    arrays, meta = {}, {}

    def put(case, **kw):
        for k, v in kw.items():
            if v is not None:
                arrays[f"{case}/{k}"] = v

    # ---- fwd + bwd cases (incl. the small fp32 plumbing configuration: batch 2, dim 64, seqlen 512) --------------------------------
    def fwd_bwd_case(name, seed, batch, dim, seqlen, width, itype, wtype, has_bias, silu,
                     init, final, uniform_w=False):
        torch.manual_seed(seed)
        x = torch.randn(batch, dim, seqlen).to(DT[itype]).requires_grad_()
        if uniform_w:
            weight = (torch.rand(dim, width) - 0.5).to(DT[wtype]).requires_grad_()
            bias = (torch.rand(dim) - 0.5).to(DT[wtype]).requires_grad_() if has_bias else None
        else:
            weight = torch.randn(dim, width).to(DT[wtype]).requires_grad_()
            bias = torch.randn(dim).to(DT[wtype]).requires_grad_() if has_bias else None
        ini = torch.randn(batch, dim, width - 1).to(DT[itype]).requires_grad_() if init else None
        act = "silu" if silu else None
        res = conv_ref(x, weight, bias, initial_states=ini, return_final_states=final, activation=act)
        if final:
            out, fs = res
            fs.retain_grad()
            # same trick as tests/test_causal_conv1d.py:117-119 to give final_states a gradient
            loss_out = out + torch.sigmoid(fs).sum(dim=-1, keepdim=True)
        else:
            out, fs, loss_out = res, None, res
        dout = torch.randn(batch, dim, seqlen).to(DT[itype])
        loss_out.backward(dout)
        dfinal = fs.grad if final else None   # exactly what autograd handed to the conv's backward
        put(name, x=f32(x), weight=f32(weight), bias=f32(bias), initial_states=f32(ini), dout=f32(dout),
            out=f32(out), final_states=f32(fs), dx=f32(x.grad), dweight=f32(weight.grad),
            dbias=f32(bias.grad) if has_bias else None,
            dinitial_states=f32(ini.grad) if init else None, dfinal_states=f32(dfinal))
        meta[name] = dict(kind="fwd_bwd", itype=itype, wtype=wtype, width=width, silu=silu,
                          has_bias=has_bias, init=init, final=final)

    fwd_bwd_case("c1_cpu_plumbing", 0, 2, 64, 512, 4, "fp32", "fp32", True, True, False, False,
                 uniform_w=True)
    k = 0
    for width in (2, 3, 4):
        for silu in (False, True):
            for itype, wtype in (("fp32", "fp32"), ("bf16", "fp32"), ("fp16", "fp32"), ("bf16", "bf16")):
                for seqlen in (1, 2, 19):
                    for init, final in ((False, False), (True, True)):
                        k += 1
                        if k % 3 != 0 and not (width == 4 and silu and itype != "fp16"):
                            continue  # thin the grid, keep width-4 SiLU complete
                        fwd_bwd_case(f"fb_w{width}_s{int(silu)}_{itype}_{wtype}_l{seqlen}_i{int(init)}",
                                     100 + k, 2, 16, seqlen, width, itype, wtype, k % 2 == 0, silu, init, final)

    # ---- seq_idx cases: the reference runs its oracle per sub-sequence ----------------
    def seqidx_case(name, seed, seqlens, pad, width, itype, silu, has_bias):
        torch.manual_seed(seed)
        batch, dim = len(seqlens), 16
        total = max(sum(s) for s in seqlens) + pad
        x = torch.randn(batch, dim, total).to(DT[itype]).requires_grad_()
        weight = torch.randn(dim, width, requires_grad=True)
        bias = torch.randn(dim, requires_grad=True) if has_bias else None
        act = "silu" if silu else None
        seq_idx = torch.full((batch, total), -1, dtype=torch.int32)
        outs = []
        for b, sl in enumerate(seqlens):
            pos, parts = 0, []
            for i, s in enumerate(sl):
                seq_idx[b, pos:pos + s] = i
                parts.append(conv_ref(x[[b], :, pos:pos + s], weight, bias, activation=act))
                pos += s
            if pos < total:  # padded tail: output defined as zero (tests/test_causal_conv1d.py:545)
                parts.append(torch.zeros(1, dim, total - pos, dtype=DT[itype]))
            outs.append(torch.cat(parts, dim=2))
        out = torch.cat(outs, dim=0)
        dout = torch.randn(batch, dim, total).to(DT[itype])
        out.backward(dout)
        put(name, x=f32(x), weight=f32(weight), bias=f32(bias), seq_idx=seq_idx.numpy(), dout=f32(dout),
            out=f32(out), dx=f32(x.grad), dweight=f32(weight.grad), dbias=f32(bias.grad) if has_bias else None)
        meta[name] = dict(kind="seq_idx", itype=itype, wtype="fp32", width=width, silu=silu,
                          has_bias=has_bias, padded=pad > 0)

    k = 0
    for width in (2, 3, 4):
        for itype in ("fp32", "bf16"):
            for pad in (0, 5):
                k += 1
                lens = [[7, 1, 2, 13], [23], [1, 1, 1, 20]] if pad == 0 else [[7, 1, 2, 9], [19], [1, 1, 1, 10]]
                if pad == 0:
                    assert len({sum(s) for s in lens}) == 1
                seqidx_case(f"si_w{width}_{itype}_p{pad}", 200 + k, lens, pad, width, itype, k % 2 == 0, k % 3 != 0)

    # ---- decode update ------------------------------------------------------------------
    def update_case(name, seed, batch, dim, seqlen, width, state_len, itype, wtype, silu, has_bias, circ):
        torch.manual_seed(seed)
        x = torch.randn(batch, dim, seqlen).to(DT[itype])
        state = torch.randn(batch, dim, state_len).to(DT[itype])
        weight = torch.randn(dim, width).to(DT[wtype])
        bias = torch.randn(dim).to(DT[wtype]) if has_bias else None
        cache = torch.randint(0, 1024, (batch,), dtype=torch.int32) if circ else None
        st = state.clone()
        out = update_ref(x, st, weight, bias, activation="silu" if silu else None, cache_seqlens=cache)
        put(name, x=f32(x), conv_state=f32(state), weight=f32(weight), bias=f32(bias),
            cache_seqlens=None if cache is None else cache.numpy(), out=f32(out), conv_state_out=f32(st))
        meta[name] = dict(kind="update", itype=itype, wtype=wtype, width=width, silu=silu,
                          has_bias=has_bias, circular=circ)

    k = 0
    for width in (2, 3, 4):
        for seqlen in (1, 4, 5):
            for circ in (False, True):
                for itype, wtype in (("fp32", "fp32"), ("bf16", "fp32"), ("fp16", "fp16"), ("bf16", "bf16")):
                    k += 1
                    if k % 2:
                        continue
                    state_len = width - 1 + (k % 5)
                    if circ and seqlen > state_len:
                        # scatter_ with duplicate indices has no defined order in torch: skip
                        state_len = seqlen + (k % 3)
                    update_case(f"up_w{width}_l{seqlen}_c{int(circ)}_{itype}_{wtype}", 300 + k, 3, 16, seqlen,
                                width, state_len, itype, wtype, k % 3 == 0, k % 4 != 0, circ)

    # ---- varlen states --------------------------------------------------------------------
    for j, (itype, state_len) in enumerate((("fp32", 20), ("bf16", 4), ("fp16", 3))):
        torch.manual_seed(400 + j)
        lens = torch.randint(1, 31, (12,))
        cu = F.pad(lens.cumsum(0), (1, 0))          # int64, like tests/test_causal_conv1d.py:332-335
        x = torch.randn(int(cu[-1]), 24).to(DT[itype])
        states = varlen_ref(x, cu, state_len)
        name = f"vs_{itype}_s{state_len}"
        put(name, x=f32(x), cu_seqlens=cu.numpy(), states=f32(states))
        meta[name] = dict(kind="varlen_states", itype=itype, state_len=state_len)

    np.savez_compressed(os.path.join(HERE, "golden.npz"), **arrays)
    with open(os.path.join(HERE, "golden.json"), "w") as f:
        json.dump({"torch": torch.__version__, "cases": meta}, f, indent=1, sort_keys=True)
    print(f"{len(meta)} cases, {sum(a.nbytes for a in arrays.values()) / 1e6:.2f} MB raw")


if __name__ == "__main__":
    if len(sys.argv) != 2:
        raise SystemExit(__doc__)
    main(sys.argv[1])
