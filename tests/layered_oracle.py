"""Slow, plain restatement of the layer-list model mechanisms, one function per mechanism, in float64 on the CPU.
It is written from the equations (below, in this file's own notation) and shares no code with the package: it takes
the weights as a dict of tensors and whole sequences, knows nothing of pages, slots, portions or batches.

Notation: T tokens, position t = 0 .. T-1; rows are tokens.  rms(v) = v / sqrt(mean(v^2) + eps).
"""
import math

import torch

F64 = torch.float64


def rms_unit(v, eps):
    return v / torch.sqrt((v * v).mean(dim=-1, keepdim=True) + eps)


def norm_around_zero(v, w, eps):
    """weight stored around zero: rms(v) * (1 + w)"""
    return rms_unit(v, eps) * (1.0 + w)


def norm_plain(v, w, eps):
    return rms_unit(v, eps) * w


def norm_in_parts(v, w, parts, eps):
    """each of `parts` equal slices of the last axis by its own root mean square, then the weight"""
    T, n = v.shape
    return rms_unit(v.reshape(T, parts, n // parts), eps).reshape(T, n) * w


def rotate_half_layout(v, positions, base, dims):
    """v [T, ..., >= dims]: dimension i < dims/2 pairs with i + dims/2; angle = position * base^(-2i/dims)."""
    half = dims // 2
    out = v.clone()
    for i in range(half):
        ang = positions.to(F64) * (base ** (-2.0 * i / dims))
        c = torch.cos(ang).reshape([-1] + [1] * (v.dim() - 2))
        s = torch.sin(ang).reshape([-1] + [1] * (v.dim() - 2))
        a, b = v[..., i], v[..., i + half]
        out[..., i] = a * c - b * s
        out[..., i + half] = b * c + a * s
    return out


def latent_attention(h, w, m, eps, shared=None):
    """h [T, width]; w: this mixer's tensors by short name; m: its sizes.  Returns (output [T, width], (latent, key_rot))
    where the pair is what a layer with kv_from reads.  `shared`: that pair from the layer kv_from names."""
    T = h.shape[0]
    H, dn, dr, dv, r = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    pos = torch.arange(T)
    q = (norm_plain(h @ w["dq"].T, w["dq.norm"], eps) @ w["uq"].T).reshape(T, H, dn + dr)
    q_plain, q_rot = q[..., :dn], rotate_half_layout(q[..., dn:], pos, m["rot"]["base"], m["rot"]["dims"])
    if shared is None:
        down = h @ w["dkv"].T
        latent = norm_plain(down[:, :r], w["dkv.norm"], eps)
        key_rot = rotate_half_layout(down[:, r:], pos, m["rot"]["base"], m["rot"]["dims"])
    else:
        latent, key_rot = shared
    keys = (latent @ w["uk"].T).reshape(T, H, dn)
    vals = (latent @ w["uv"].T).reshape(T, H, dv)
    out = torch.zeros(T, H, dv, dtype=F64)
    for i in range(T):                                   # query i sees keys 0 .. i
        for hh in range(H):
            sc = (keys[:i + 1, hh] @ q_plain[i, hh] + key_rot[:i + 1] @ q_rot[i, hh]) * m["scale"]
            p = torch.softmax(sc, dim=0)
            out[i, hh] = p @ vals[:i + 1, hh]
    gated = out.reshape(T, H * dv) * torch.sigmoid(h @ w["g"].T)
    return gated @ w["o"].T, (latent, key_rot)


def mamba2(h, w, m, eps):
    T = h.shape[0]
    H, P, N, G, taps, parts = m["heads"], m["vdim"], m["state"], m["groups"], m["conv"], m["norm_groups"]
    inner = H * P
    proj = h @ w["in"].T
    z, xbc, dt = proj[:, :inner], proj[:, inner:2 * inner + 2 * G * N], proj[:, 2 * inner + 2 * G * N:]
    conv = torch.zeros_like(xbc)
    for t in range(T):
        acc = w["conv.b"].clone()
        for k in range(taps):                            # last column is the current token's
            src = t - (taps - 1) + k
            if src >= 0:
                acc = acc + w["conv"][:, k] * xbc[src]
        conv[t] = acc
    xbc = conv * torch.sigmoid(conv)
    x = xbc[:, :inner].reshape(T, H, P)
    B = xbc[:, inner:inner + G * N].reshape(T, G, N)
    C = xbc[:, inner + G * N:].reshape(T, G, N)
    step = torch.log1p(torch.exp(dt + w["dt_bias"]))
    rate = torch.exp(w["A_log"])
    y = torch.zeros(T, H, P, dtype=F64)
    for hh in range(H):
        grp = hh // (H // G)
        S = torch.zeros(N, P, dtype=F64)
        for t in range(T):
            S = math.exp(-float(rate[hh]) * float(step[t, hh])) * S + step[t, hh] * torch.outer(B[t, grp], x[t, hh])
            y[t, hh] = S.T @ C[t, grp] + w["D"][hh] * x[t, hh]
    gated = y.reshape(T, inner) * (z * torch.sigmoid(z))
    return norm_in_parts(gated, w["norm"], parts, eps) @ w["o"].T


def squared_relu_ff(h, w):
    return torch.clamp(h @ w["up"].T, min=0.0) ** 2 @ w["down"].T


def sub(tensors, prefix):
    return {k[len(prefix):]: v.to(F64) for k, v in tensors.items() if k.startswith(prefix)}


def model_logits(tensors, config, tokens, residual_out=None):
    """Logits [T, vocab] of one whole sequence."""
    eps = config["norm"]["eps"]
    W = {k: v.to(F64) for k, v in tensors.items()}
    x = W["embed"][torch.tensor(tokens)]
    caches = {}
    for i, layer in enumerate(config["layers"]):
        p = f"l{i}."
        h = norm_around_zero(x, W[p + "norm1"], eps)
        if layer["type"] == "latent_attention":
            src = layer["mixer"].get("kv_from")
            y, caches[i] = latent_attention(h, sub(tensors, p + "mix."), layer["mixer"], eps, None if src is None else caches[src])
        else:
            y = mamba2(h, sub(tensors, p + "mix."), layer["mixer"], eps)
        x = x + norm_around_zero(y, W[p + "norm1b"], eps)
        if layer.get("mlp"):
            h = norm_around_zero(x, W[p + "norm2"], eps)
            x = x + norm_around_zero(squared_relu_ff(h, sub(tensors, p + "mlp.")), W[p + "norm2b"], eps)
        if residual_out is not None:
            residual_out.append(x.clone())
    lg = norm_around_zero(x, W["final.norm"], eps) @ W["head"].T
    cap = config.get("logit_softcap")
    return cap * torch.tanh(lg / cap) if cap else lg


def logit_error(got, want):
    """Per row: root mean square of the difference (mean taken off) over the root mean square of the wanted logits."""
    d = got.to(F64) - want.to(F64)
    d = d - d.mean(dim=-1, keepdim=True)
    return d.pow(2).mean(dim=-1).sqrt() / want.to(F64).pow(2).mean().sqrt()
