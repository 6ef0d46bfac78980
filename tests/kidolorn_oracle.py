"""Plain, slow statement of the Kidolorn decoder, one function per mechanism, in torch on the CPU.

It is the checker of the tests and shares nothing with the product path: it reads a dictionary of tensors keyed by
the model's tensor names and a configuration dictionary with the keys of the model's config.json, and recomputes
every position from the whole token sequence (no cache, no state carried between calls).

Notation: W is the model width, t a position counted from 0, h the input a sublayer reads.
"""
import math

import torch


def rms_unit(x, eps):
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def scalar_norm(x, g, eps):
    """RMS norm whose gain is one number for all coordinates."""
    return rms_unit(x, eps) * g


def canon(h, w):
    """h + causal depthwise convolution of h over time.  h [T, W], w [W, taps]; tap j multiplies h at t - taps + 1 + j."""
    T, taps = h.shape[0], w.shape[1]
    out = h.clone()
    for j in range(taps):
        back = taps - 1 - j
        if back >= T:
            continue
        shifted = torch.zeros_like(h)
        shifted[back:] = h[:T - back] if back else h
        out = out + shifted * w[:, j]
    return out


def silu(x):
    return x * torch.sigmoid(x)


def lightning(h, P, mx, eps):
    """Linear attention with one fixed decay per head: S_t = a S_{t-1} + k_t v_t^T, o_t = S_t^T q_t."""
    H, d, dv = mx["heads"], mx["dim"], mx["vdim"]
    T = h.shape[0]
    q = silu(h @ P["q"].T).view(T, H, d)
    k = silu(h @ P["k"].T).view(T, H, d)
    v = silu(h @ P["v"].T).view(T, H, dv)
    o = torch.zeros(T, H, dv, dtype=h.dtype)
    for hd in range(H):
        a = float(mx["decay"][hd])
        S = torch.zeros(d, dv, dtype=h.dtype)
        for t in range(T):
            S = a * S + torch.outer(k[t, hd], v[t, hd])
            o[t, hd] = S.T @ q[t, hd]
    o = rms_unit(o.reshape(T, H * dv), eps) * P["norm"]
    o = o * torch.sigmoid(h @ P["g"].T)
    return o @ P["o"].T


def mingru(h, P, mx):
    """Gated recurrence whose gates read only the current token."""
    T = h.shape[0]
    z = torch.sigmoid(h @ P["z"].T + P["z.b"])
    u = h @ P["x"].T + P["x.b"]
    cand = torch.where(u >= 0, u + 0.5, torch.sigmoid(u))
    S = torch.zeros(mx["width"], dtype=h.dtype)
    out = torch.zeros(T, mx["width"], dtype=h.dtype)
    gate = silu(h @ P["g"].T)
    for t in range(T):
        S = (1 - z[t]) * S + z[t] * cand[t]
        out[t] = S * gate[t]
    return out @ P["o"].T


def rotate(x, pos, base, dims):
    """Rotary position on the first `dims` coordinates of the last axis; coordinate i pairs with i + dims/2."""
    half = dims // 2
    i = torch.arange(half, dtype=torch.float64)
    f = base ** (-2.0 * i / dims)
    a = pos.to(torch.float64)[:, None] * f[None, :]
    cos, sin = a.cos().to(x.dtype), a.sin().to(x.dtype)
    while cos.dim() < x.dim():
        cos, sin = cos.unsqueeze(1), sin.unsqueeze(1)
    u, v = x[..., :half], x[..., half:dims]
    return torch.cat([u * cos - v * sin, v * cos + u * sin, x[..., dims:]], -1)


def latent_kv(h, P, mx, eps):
    """What a latent-attention layer caches: the normed latent c [T, kv_rank] and the rotated shared key part [T, rot_dim]."""
    T = h.shape[0]
    r, dr = mx["kv_rank"], mx["rot_dim"]
    d = h @ P["dkv"].T
    c = rms_unit(d[:, :r], eps) * P["dkv.norm"]
    kr = rotate(d[:, r:r + dr], torch.arange(T), mx["rot"]["base"], mx["rot"]["dims"])
    return c, kr


def latent_attention(h, P, mx, c, kr):
    """Causal softmax attention over keys rebuilt from the latent, with a sink in the denominator and an output gate."""
    T = h.shape[0]
    H, d, dr, dv, r = mx["heads"], mx["dim"], mx["rot_dim"], mx["vdim"], mx["kv_rank"]
    q = (h @ P["q"].T).view(T, H, d + dr)
    qn = q[..., :d]
    qr = rotate(q[..., d:], torch.arange(T), mx["rot"]["base"], mx["rot"]["dims"])
    kn = (c @ P["uk"].T).view(T, H, d)
    v = (c @ P["uv"].T).view(T, H, dv)
    out = torch.zeros(T, H, dv, dtype=h.dtype)
    causal = torch.tril(torch.ones(T, T, dtype=torch.bool))
    for hd in range(H):
        s = (qn[:, hd] @ kn[:, hd].T + qr[:, hd] @ kr.T) * mx["scale"]
        s = s.masked_fill(~causal, -math.inf)
        m = torch.maximum(s.max(-1, keepdim=True).values, P["sink"][hd].expand(T, 1))
        e = torch.exp(s - m)
        den = e.sum(-1, keepdim=True) + torch.exp(P["sink"][hd] - m)
        out[:, hd] = (e / den) @ v[:, hd]
    out = out.reshape(T, H * dv) * torch.sigmoid(h @ P["g"].T)
    return out @ P["o"].T


def gated_unit(h, gate, up, down, limit, gb=None, ub=None, db=None):
    """min / clamp limited gate and up branches: y = g sigmoid(1.702 g) (u + 1), then the down projection."""
    g = h @ gate.T
    u = h @ up.T
    if gb is not None:
        g, u = g + gb, u + ub
    g = torch.clamp(g, max=limit)
    u = torch.clamp(u, -limit, limit)
    y = (g * torch.sigmoid(1.702 * g) * (u + 1)) @ down.T
    return y + db if db is not None else y


def dense_ff(h, P, ml):
    return gated_unit(h, P["gate"], P["up"], P["down"], ml["limit"], P["gate.b"], P["up.b"], P["down.b"])


def route(h, router, top):
    """Indices of the `top` largest router logits per token and the softmax over those logits only."""
    z = h.float() @ router.float().T if h.dtype != torch.float64 else h @ router.T
    val, idx = torch.topk(z, top, dim=-1)
    return idx, torch.softmax(val, -1).to(h.dtype)


def moe_ff(h, P, ml):
    idx, w = route(h, P["router"], ml["router"]["top"])
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for j in range(idx.shape[1]):
            e = int(idx[t, j])
            y = gated_unit(h[t:t + 1], P[f"e{e}.gate"], P[f"e{e}.up"], P[f"e{e}.down"], ml["expert"]["limit"])
            out[t] += w[t, j] * y[0]
    return out


def _sub(tensors, prefix, dtype):
    n = len(prefix)
    return {k[n:]: v.to(dtype) for k, v in tensors.items() if k.startswith(prefix)}


def forward(cfg, tensors, tokens, dtype=torch.float64, layers_out=None):
    """Logits [T, vocab] of one sequence; layers_out (a list) receives the residual stream after every layer."""
    eps = cfg["norm"]["eps"]
    taps = cfg["canon"]["taps"] if cfg.get("canon") else 0
    tok = torch.as_tensor(tokens, dtype=torch.long)
    x = tensors["embed"].to(dtype)[tok]
    kept = {}
    for i, ly in enumerate(cfg["layers"]):
        pre = f"l{i}."
        g = {k: tensors[pre + k].to(dtype) for k in ("norm1", "norm1b", "norm2", "norm2b") if pre + k in tensors}
        mx, P = ly["mixer"], _sub(tensors, pre + "mix.", dtype)
        h = scalar_norm(x, g["norm1"], eps)
        if taps >= 1:
            h = canon(h, tensors[pre + "canon1"].to(dtype))
        if ly["type"] == "lightning":
            y = lightning(h, P, mx, eps)
        elif ly["type"] == "mingru":
            y = mingru(h, P, mx)
        elif ly["type"] == "latent_attention":
            if "kv_from" in mx and mx["kv_from"] is not None:
                c, kr = kept[mx["kv_from"]]
            else:
                c, kr = kept[i] = latent_kv(h, P, mx, eps)
            y = latent_attention(h, P, mx, c, kr)
        else:
            raise ValueError(ly["type"])
        x = x + scalar_norm(y, g["norm1b"], eps)
        ml = ly.get("mlp")
        if ml is not None:
            h = scalar_norm(x, g["norm2"], eps)
            if taps >= 1:
                h = canon(h, tensors[pre + "canon2"].to(dtype))
            M = _sub(tensors, pre + "mlp.", dtype)
            y = dense_ff(h, M, ml) if ml["kind"] == "dense" else moe_ff(h, M, ml)
            x = x + scalar_norm(y, g["norm2b"], eps)
        if layers_out is not None:
            layers_out.append(x.clone())
    x = scalar_norm(x, tensors["final.norm"].to(dtype), eps)
    return x @ tensors["head"].to(dtype).T
