"""float64 PyTorch statement of the op for checks at sizes the CPU oracle is too slow for.

Test infrastructure only.  A shifted-sum formulation (no F.conv1d, so no cuDNN / TF32):
out[b,c,t] = act(bias[c] + sum_k weight[c,k] * xp[b,c,t+k]) with xp = [initial_states | x],
taps masked by seq_idx equality, padded tokens (seq_idx < 0) forced to zero.  Gradients
come from autograd on this expression.  It is itself checked against the CPU oracle in
tests/test_torch_ref_cpu.py.
"""
import torch


def conv_ref64(x, weight, bias=None, seq_idx=None, initial_states=None, return_final_states=False,
               activation=None):
    B, D, L = x.shape
    W = weight.shape[1]
    x = x.double()
    weight = weight.double()
    head = initial_states.double() if initial_states is not None else x.new_zeros(B, D, W - 1)
    xp = torch.cat([head, x], dim=-1)
    out = x.new_zeros(B, D, L) if bias is None else bias.double()[None, :, None].expand(B, D, L)
    if seq_idx is not None:
        sp = torch.cat([seq_idx.new_full((B, W - 1), -1), seq_idx], dim=-1)
    for k in range(W):
        tap = xp[..., k:k + L] * weight[:, k][None, :, None]
        if seq_idx is not None:
            tap = torch.where((sp[:, k:k + L] == seq_idx)[:, None, :], tap, torch.zeros_like(tap))
        out = out + tap
    if activation in ("silu", "swish"):
        out = out * torch.sigmoid(out)
    if seq_idx is not None:
        out = torch.where((seq_idx < 0)[:, None, :], torch.zeros_like(out), out)
    if return_final_states:
        return out, xp[..., L:]
    return out


def conv_grads64(x, weight, bias, dout, seq_idx=None, initial_states=None, dfinal_states=None, activation=None):
    """Returns dict(out, final_states, dx, dweight, dbias, dinitial_states) in float64."""
    xd = x.detach().double().requires_grad_()
    wd = weight.detach().double().requires_grad_()
    bd = bias.detach().double().requires_grad_() if bias is not None else None
    idd = initial_states.detach().double().requires_grad_() if initial_states is not None else None
    want_final = dfinal_states is not None
    res = conv_ref64(xd, wd, bd, seq_idx, idd, want_final, activation)
    out, fs = res if want_final else (res, None)
    loss = (out * dout.double()).sum()
    if want_final:
        loss = loss + (fs * dfinal_states.double()).sum()
    loss.backward()
    return dict(out=out.detach(), final_states=None if fs is None else fs.detach(), dx=xd.grad, dweight=wd.grad,
                dbias=None if bd is None else bd.grad, dinitial_states=None if idd is None else idd.grad)
