"""A plain, slow restatement of the Motolix decoder in numpy float64: one function per mechanism, whole sequences at once for
the position-wise parts and token by token for the recurrence.  It shares nothing with the engine; tests compare the
engine's logits (and, through models cut short, its residual stream) against it.

Notation: x is the residual stream [T, W]; a model is (cfg, tensors) with cfg the parsed config.json and tensors a dict
name -> float array.  Positions count from 0.
"""
import numpy as np


def layer_norm(x, w, b, eps):
    mu = x.mean(-1, keepdims=True)
    var = ((x - mu) ** 2).mean(-1, keepdims=True)
    return (x - mu) / np.sqrt(var + eps) * w + b


def unit_rms(x, eps):
    return x / np.sqrt((x * x).mean(-1, keepdims=True) + eps)


def gelu_tanh(z):
    return 0.5 * z * (1.0 + np.tanh(np.sqrt(2.0 / np.pi) * (z + 0.044715 * z ** 3)))


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def rotary_frequencies(rot):
    """f_i = base^(-2i/n) for the n/2 coordinate pairs; with `scaling`, long wavelengths are stretched by `factor`, short ones
    kept, and the band between original/low and original/high blended linearly in original/wavelength."""
    n = int(rot["dims"])
    f = float(rot["base"]) ** (-2.0 * np.arange(n // 2) / n)
    sc = rot.get("scaling")
    if not sc:
        return f
    out = np.empty_like(f)
    for i, fi in enumerate(f):
        wavelength = 2.0 * np.pi / fi
        if wavelength < sc["original"] / sc["high"]:
            out[i] = fi
        elif wavelength > sc["original"] / sc["low"]:
            out[i] = fi / sc["factor"]
        else:
            s = (sc["original"] / wavelength - sc["low"]) / (sc["high"] - sc["low"])
            out[i] = (1.0 - s) * fi / sc["factor"] + s * fi
    return out


def rotate(v, positions, f, sign=1.0):
    """v [T, heads, n]: coordinates i and i + len(f) (i < len(f)) of every head turn by sign * position * f_i; coordinates from
    2 len(f) on pass unchanged."""
    h = len(f)
    out = np.array(v, dtype=np.float64, copy=True)
    for t, p in enumerate(positions):
        ang = sign * p * f
        c, s = np.cos(ang), np.sin(ang)
        a, b = v[t, :, :h], v[t, :, h:2 * h]
        out[t, :, :h] = a * c - b * s
        out[t, :, h:2 * h] = b * c + a * s
    return out


def sigmoid_attention(h, tens, p, m):
    """Grouped-query attention whose values are the unrotated keys and whose weights are sigmoid(score * temp + pb), one
    weight per visible key, not normalised.  Biases on q, k and the output projection."""
    T = h.shape[0]
    H, G, d = m["heads"], m["kv_heads"], m["dim"]
    q = (h @ tens[p + "q"].T + tens[p + "q.b"]).reshape(T, H, d)
    k = (h @ tens[p + "k"].T + tens[p + "k.b"]).reshape(T, G, d)
    v = k.copy()
    f = rotary_frequencies(m["rot"])
    pos = np.arange(T)
    q, k = rotate(q, pos, f), rotate(k, pos, f)
    out = np.zeros((T, H, m["vdim"]))
    for i in range(T):
        for hd in range(H):
            g = hd // (H // G)
            for j in range(i + 1):
                s = float(q[i, hd] @ k[j, g]) * m["scale"] * tens[p + "temp"][hd]
                out[i, hd] += sigmoid(s + tens[p + "pb"][hd]) * v[j, g]
    return out.reshape(T, -1) @ tens[p + "o"].T + tens[p + "o.b"]


def softmax_attention_rotated_values(h, tens, p, m, eps):
    """Grouped-query softmax attention.  q and k are normalised over the whole projection (all heads at once) with gain vectors,
    then rotated; the value of position j is rotated by j over all its coordinates, and a head's output at position i is
    rotated back by i."""
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = (unit_rms(h @ tens[p + "q"].T, eps) * tens[p + "q.norm"]).reshape(T, H, d)
    k = (unit_rms(h @ tens[p + "k"].T, eps) * tens[p + "k.norm"]).reshape(T, G, d)
    v = (h @ tens[p + "v"].T).reshape(T, G, dv)
    pos = np.arange(T)
    f = rotary_frequencies(m["rot"])
    q, k = rotate(q, pos, f), rotate(k, pos, f)
    fv = float(m["rot"]["base"]) ** (-2.0 * np.arange(dv // 2) / dv)
    v = rotate(v, pos, fv)
    out = np.zeros((T, H, dv))
    for i in range(T):
        for hd in range(H):
            g = hd // (H // G)
            s = np.array([float(q[i, hd] @ k[j, g]) * m["scale"] for j in range(i + 1)])
            w = np.exp(s - s.max())
            w /= w.sum()
            out[i, hd] = w @ v[:i + 1, g]
    out = rotate(out, pos, fv, sign=-1.0)
    return out.reshape(T, -1) @ tens[p + "o"].T


def gated_linear_attention(h, tens, p, m, eps, state=None):
    """Per head a matrix S [dim, vdim]: S <- diag(a_t) S + k_t v_t^T, o_t = S^T q_t, q scaled by dim^(-1/2), the decay
    a_t = sigmoid(z_t)^(1/tau) with z_t from a two-step projection with a bias.  o is normalised per head (gain shared by the
    heads), gated by silu of a projection of h, and projected."""
    T = h.shape[0]
    H, d, dv = m["heads"], m["dim"], m["vdim"]
    q = (h @ tens[p + "q"].T).reshape(T, H, d) * d ** -0.5
    k = (h @ tens[p + "k"].T).reshape(T, H, d)
    v = (h @ tens[p + "v"].T).reshape(T, H, dv)
    z = (h @ tens[p + "a1"].T) @ tens[p + "a2"].T + tens[p + "a2.b"]
    a = (sigmoid(z) ** (1.0 / m["tau"])).reshape(T, H, d)
    S = np.zeros((H, d, dv)) if state is None else state
    o = np.zeros((T, H, dv))
    for t in range(T):
        for hd in range(H):
            S[hd] = a[t, hd][:, None] * S[hd] + np.outer(k[t, hd], v[t, hd])
            o[t, hd] = S[hd].T @ q[t, hd]
    o = unit_rms(o, eps) * tens[p + "norm"]
    gate = h @ tens[p + "g"].T
    return (o.reshape(T, -1) * gate * sigmoid(gate)) @ tens[p + "o"].T


def feed_forward(h, tens, p):
    return (gelu_tanh(h @ tens[p + "gate"].T) * (h @ tens[p + "up"].T)) @ tens[p + "down"].T


def layer_order(cfg):
    """(layer index, loop pass or None) of every layer run: the looped stretch repeated, its first layer marked with the pass."""
    n = len(cfg["layers"])
    lp = cfg.get("loop")
    if not lp:
        return [(i, None) for i in range(n)]
    runs = [(i, None) for i in range(lp["start"])]
    for t in range(lp["times"]):
        runs += [(i, t if i == lp["start"] else None) for i in range(lp["start"], lp["stop"])]
    return runs + [(i, None) for i in range(lp["stop"], n)]


def forward(cfg, tens, tokens, layers_out=None):
    """Logits [T, vocab] of a whole sequence; layers_out (a list) receives the residual stream after every layer run."""
    tens = {k: np.asarray(v, np.float64) for k, v in tens.items()}
    eps = cfg["norm"]["eps"]
    x = tens["embed"][np.asarray(tokens)] * cfg["embedding"]["scale"]
    x0 = x.copy()

    def ln(v, name):
        return layer_norm(v, tens[name], tens[name + ".b"], eps)
    for i, loop_pass in layer_order(cfg):
        ly, p = cfg["layers"][i], f"l{i}."
        if loop_pass is not None:
            x = np.concatenate([x, x0], -1) @ tens["loop.in"].T + tens["loop.step"][loop_pass]
        h = ln(x, p + "norm1")
        if ly["type"] == "attention":
            y = sigmoid_attention(h, tens, p + "mix.", ly["mixer"])
        else:
            m = ly["mixer"]
            y = (m["left_scale"] * softmax_attention_rotated_values(h, tens, p + "mix.left.", m["left"], eps)
                 + m["right_scale"] * gated_linear_attention(h, tens, p + "mix.right.", m["right"], eps))
        x = x + ln(y, p + "norm1b")
        if ly.get("mlp"):
            x = x + ln(feed_forward(ln(x, p + "norm2"), tens, p + "mlp."), p + "norm2b")
        if layers_out is not None:
            layers_out.append(x.copy())
    return ln(x, "final.norm") @ tens["head"].T * cfg["logit_scale"]
