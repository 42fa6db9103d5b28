"""Slow, plain restatement of the Sunesun mechanisms in float64 on the CPU, one function per mechanism, written from
the equations in this file's own notation.  It shares no code with the package: weights come as a dict of tensors,
sequences whole; it knows nothing of pages, slots, portions, batches or kernels.

Notation: T tokens at positions t = 0 .. T-1; rms(v) = v / sqrt(mean(v^2) + eps).
"""
import math

import torch

F64 = torch.float64


def rms_weighted(v, w, eps):
    return v / torch.sqrt((v * v).mean(dim=-1, keepdim=True) + eps) * w


def rotary_table(rot, T):
    """cos, sin [T, dims/2] for the pairs (2i, 2i+1).  Base frequencies b^(-2i/dims); with `scaling` the slow ones are
    divided by `factor`, the fast ones kept, a linear ramp between; cos and sin grow by 0.1 ln(factor) + 1."""
    dims, base = rot["dims"], rot["base"]
    freq = [base ** (-2.0 * i / dims) for i in range(dims // 2)]
    grow = 1.0
    sc = rot.get("scaling")
    if sc:
        def where(turns):
            return dims * math.log(sc["original"] / (2.0 * math.pi * turns)) / (2.0 * math.log(base))
        lo = max(math.floor(where(sc["fast"])), 0)
        hi = min(math.ceil(where(sc["slow"])), dims - 1)
        for i in range(dims // 2):
            ramp = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
            freq[i] = freq[i] / sc["factor"] * ramp + freq[i] * (1.0 - ramp)
        grow = 0.1 * math.log(sc["factor"]) + 1.0
    ang = torch.arange(T, dtype=F64)[:, None] * torch.tensor(freq, dtype=F64)[None, :]
    return torch.cos(ang) * grow, torch.sin(ang) * grow


def rotate_interleaved(v, cos, sin):
    """v [T, heads, dim]: the first 2 * cos.shape[1] dimensions of every head, pairs (2i, 2i + 1)."""
    out = v.clone()
    for i in range(cos.shape[1]):
        a, b = v[:, :, 2 * i], v[:, :, 2 * i + 1]
        c, s = cos[:, i:i + 1], sin[:, i:i + 1]
        out[:, :, 2 * i] = a * c - b * s
        out[:, :, 2 * i + 1] = b * c + a * s
    return out


def windowed_attention(h, w, m):
    """h [T, width] -> [T, width].  Values are the keys as projected (before rotation)."""
    T = h.shape[0]
    H, G, d = m["heads"], m["kv_heads"], m["dim"]
    q = (h @ w["q"].T).reshape(T, H, d)
    k = (h @ w["k"].T).reshape(T, G, d)
    values = k
    rot = m.get("rot")
    if rot and rot["dims"]:
        cos, sin = rotary_table(rot, T)
        q, k = rotate_interleaved(q, cos, sin), rotate_interleaved(k, cos, sin)
    window = (m.get("mask") or {}).get("size") or T + 1
    cap = m.get("softcap")
    out = torch.zeros(T, H, d, dtype=F64)
    for i in range(T):
        first = max(0, i - window + 1)
        for hh in range(H):
            g = hh // (H // G)
            sc = (k[first:i + 1, g] @ q[i, hh]) * m["scale"]
            if cap:
                sc = cap * torch.tanh(sc / cap)
            out[i, hh] = torch.softmax(sc, dim=0) @ values[first:i + 1, g]
    return out.reshape(T, H * d) @ w["o"].T


def route(scores, r):
    """scores [experts] of one token -> list of chosen expert indices, best first."""
    E, top = r["experts"], r["top"]
    grp = r.get("groups") or {"count": 1, "keep": 1}
    per = E // grp["count"]
    gscore = []
    for g in range(grp["count"]):
        best = sorted((float(scores[g * per + i]) for i in range(per)), reverse=True)[:2]
        gscore.append(sum(best))
    kept = sorted(range(grp["count"]), key=lambda g: (-gscore[g], g))[:grp["keep"]]
    eligible = [e for e in range(E) if e // per in kept]
    return sorted(eligible, key=lambda e: (-float(scores[e]), e))[:top]


def routed_experts(h, w, m):
    T = h.shape[0]
    s = torch.sigmoid(h @ w["router"].T)
    out = torch.zeros_like(h)
    for t in range(T):
        for e in route(s[t], m["router"]):
            hidden = torch.clamp(w[f"e{e}.up"] @ h[t], min=0.0) ** 2
            out[t] += s[t, e] * (w[f"e{e}.down"] @ hidden)
    return out


def hyper_read(copies, w_in):
    return sum(w_in[s] * copies[s] for s in range(len(copies)))


def hyper_write(copies, mix, w_out, mult, y):
    S = len(copies)
    return [sum(mix[s, t] * copies[s] for s in range(S)) + mult * w_out[t] * y for t in range(S)]


def sub(tensors, prefix):
    return {k[len(prefix):]: v.to(F64) for k, v in tensors.items() if k.startswith(prefix)}


def model_logits(tensors, config, tokens, residual_out=None):
    """Logits [T, vocab] of one whole sequence; residual_out collects the summed copies after every layer."""
    eps = config["norm"]["eps"]
    W = {k: v.to(F64) for k, v in tensors.items()}
    S = config.get("streams") or 0
    mult = config.get("residual_mult", 1.0)
    x0 = W["embed"][torch.tensor(tokens)] * (config.get("embedding") or {}).get("scale", 1.0)
    copies = [x0.clone() for _ in range(max(S, 1))]
    for i, layer in enumerate(config["layers"]):
        j = layer.get("weights_of", i)
        p = f"l{i if j is None else j}."
        parts = [("1", lambda h: windowed_attention(h, sub(tensors, p + "mix."), layer["mixer"]))]
        if layer.get("mlp"):
            parts.append(("2", lambda h: routed_experts(h, sub(tensors, p + "mlp."), layer["mlp"])))
        for q, fn in parts:
            if S:
                u = hyper_read(copies, W[p + f"hc{q}.in"])
                y = fn(rms_weighted(u, W[p + "norm" + q], eps))
                copies = hyper_write(copies, W[p + f"hc{q}.mix"], W[p + f"hc{q}.out"], mult, y)
            else:
                copies = [copies[0] + mult * fn(rms_weighted(copies[0], W[p + "norm" + q], eps))]
        if residual_out is not None:
            residual_out.append(sum(copies))
    return rms_weighted(sum(copies), W["final.norm"], eps) @ W["head"].T


def logit_error(got, want):
    """Per row: root mean square of the difference (mean taken off) over the root mean square of the wanted logits."""
    d = got.to(F64) - want.to(F64)
    d = d - d.mean(dim=-1, keepdim=True)
    return d.pow(2).mean(dim=-1).sqrt() / want.to(F64).pow(2).mean().sqrt()
