"""A plain, slow restatement of the Vumedra decoder, one function per mechanism.

It shares no code with the library: tensors come in as a dict name -> torch
tensor, the configuration as the parsed config.json, and everything runs on the
CPU in one dtype (float64 by default), token by token where the design has a
recurrence.  ``forward`` returns logits for a whole sequence and, optionally,
the residual stream after every layer.

Notation: T tokens, D width, H heads, G key/value heads, K key channels per
head, V value channels per head.
"""
from __future__ import annotations

import math

import torch


def rms(x, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def scalar_norm(x, g, eps):
    """RMS norm with one learned number for all channels."""
    return rms(x, eps) * g.reshape(())


def gelu_tanh(z):
    return 0.5 * z * (1 + torch.tanh(math.sqrt(2 / math.pi) * (z + 0.044715 * z ** 3)))


def softplus(z):
    return torch.where(z > 30, z, torch.log1p(torch.exp(torch.clamp(z, max=30))))


def logsigmoid(z):
    return -softplus(-z)


# ---------------------------------------------------------------------------------------------------------
def embedding(tokens, w, cfg, dtype, first_position=0, before=None):
    """Token row + bigram row + sinusoidal position.  ``before``: the token ahead of tokens[0] (None: tokens[0]
    opens the sequence)."""
    D = cfg["width"]
    big = cfg["embedding"]["bigram"]
    T = len(tokens)
    x = w["embed"][torch.as_tensor(tokens)].to(dtype).clone()
    for t, tok in enumerate(tokens):
        prev = before if t == 0 else tokens[t - 1]
        row = big["buckets"] if prev is None else (prev * big["mul_prev"] + tok * big["mul_cur"]) % big["buckets"]
        x[t] += w["bigram"][row].to(dtype)
    i = torch.arange(0, D, 2, dtype=torch.float64)
    freq = 10000.0 ** (-i / D)
    p = torch.arange(first_position, first_position + T, dtype=torch.float64)
    ang = p[:, None] * freq[None, :]
    pe = torch.zeros(T, D, dtype=torch.float64)
    pe[:, 0::2] = torch.sin(ang)[:, :(D + 1) // 2]
    pe[:, 1::2] = torch.cos(ang)[:, :D // 2]
    return x + pe.to(dtype)


# ---------------------------------------------------------------------------------------------------------
def attend_with_sink(q, k, v, scale, q_pos, k_pos, sink=True):
    """q [Tq, H, K], k [Tk, G, K], v [Tk, G, V]: causal by the positions given; with ``sink`` the denominator is
    1 + sum exp(s).  Returns [Tq, H, V]."""
    H, G = q.shape[1], k.shape[1]
    out = torch.zeros(q.shape[0], H, v.shape[2], dtype=q.dtype)
    for head in range(H):
        g = head // (H // G)
        s = (q[:, head] @ k[:, g].T) * scale
        s = s.masked_fill(k_pos[None, :] > q_pos[:, None], float("-inf"))
        if sink:
            e = torch.exp(s)
            p = e / (1 + e.sum(-1, keepdim=True))
        else:
            p = torch.softmax(s, -1)
        out[:, head] = p @ v[:, g]
    return out


def sink_attention(h, w, pre, mix, eps, positions):
    """Causal softmax attention whose denominator holds one more term, exp(0): a key that every query sees,
    with score zero and no value.  Queries and keys are RMS-normed per head; the query grows with the
    logarithm of its position, in steps."""
    H, K = mix["heads"], mix["dim"]
    G, V = mix.get("kv_heads", H), mix.get("vdim", K)
    T = h.shape[0]
    q = (h @ w[pre + "q"].T + w[pre + "q.b"]).view(T, H, K)
    k = (h @ w[pre + "k"].T + w[pre + "k.b"]).view(T, G, K)
    v = (h @ w[pre + "v"].T + w[pre + "v.b"]).view(T, G, V)
    q = rms(q, eps) * w[pre + "q.norm"]
    k = rms(k, eps) * w[pre + "k.norm"]
    temp = mix.get("q_temp")
    if temp:
        steps = torch.floor((positions.to(torch.float64) + 1) / temp["every"])
        q = q * (1 + temp["coef"] * torch.log(steps + 1)).to(h.dtype)[:, None, None]
    out = attend_with_sink(q, k, v, mix["scale"], positions, positions)
    return out.reshape(T, H * V) @ w[pre + "o"].T


def mlstm(h, w, pre, mix, eps):
    """Matrix memory with exponential input gate, kept in range by a running maximum that starts at zero."""
    H, K, V, cap = mix["heads"], mix["dim"], mix.get("vdim", mix["dim"]), mix["gate_cap"]
    T = h.shape[0]
    q = (h @ w[pre + "q"].T).view(T, H, K) * K ** -0.5
    k = (h @ w[pre + "k"].T).view(T, H, K)
    v = (h @ w[pre + "v"].T).view(T, H, V)
    gi = cap * torch.tanh((h @ w[pre + "i"].T + w[pre + "i.b"]) / cap)
    gf = logsigmoid(cap * torch.tanh((h @ w[pre + "f"].T + w[pre + "f.b"]) / cap))
    S = torch.zeros(H, K, V, dtype=h.dtype)
    n = torch.zeros(H, K, dtype=h.dtype)
    m = torch.zeros(H, dtype=h.dtype)
    out = torch.zeros(T, H, V, dtype=h.dtype)
    for t in range(T):
        m_new = torch.maximum(gf[t] + m, gi[t])
        keep, take = torch.exp(gf[t] + m - m_new), torch.exp(gi[t] - m_new)
        S = keep[:, None, None] * S + take[:, None, None] * k[t][:, :, None] * v[t][:, None, :]
        n = keep[:, None] * n + take[:, None] * k[t]
        m = m_new
        num = torch.einsum("hkv,hk->hv", S, q[t])
        den = torch.maximum((n * q[t]).sum(-1).abs(), torch.exp(-m)) + 1e-6
        out[t] = num / den[:, None]
    y = rms(out, eps).reshape(T, H * V) * w[pre + "norm"] * torch.sigmoid(h @ w[pre + "g"].T)
    return y @ w[pre + "o"].T


def rglru(h, w, pre, mix):
    """Two branches: a gate y, and a short causal convolution followed by a gated diagonal recurrence."""
    C, B = mix["width"], mix["blocks"]
    T = h.shape[0]
    y = gelu_tanh(h @ w[pre + "y"].T + w[pre + "y.b"])
    xin = h @ w[pre + "x"].T + w[pre + "x.b"]
    taps = w[pre + "conv"].shape[1]
    padded = torch.cat([torch.zeros(taps - 1, C, dtype=h.dtype), xin], 0)
    u = w[pre + "conv.b"].expand(T, C).clone()
    for j in range(taps):
        u = u + padded[j:j + T] * w[pre + "conv"][:, j]
    ub = u.view(T, B, C // B)
    r = torch.sigmoid(torch.einsum("boi,tbi->tbo", w[pre + "ra"], ub) + w[pre + "ra.b"]).reshape(T, C)
    i = torch.sigmoid(torch.einsum("boi,tbi->tbo", w[pre + "ri"], ub) + w[pre + "ri.b"]).reshape(T, C)
    log_a = -8.0 * r * softplus(w[pre + "lam"])
    a = torch.exp(log_a)
    S = torch.zeros(C, dtype=h.dtype)
    out = torch.zeros(T, C, dtype=h.dtype)
    for t in range(T):
        S = a[t] * S + torch.sqrt(1 - a[t] ** 2) * i[t] * u[t]
        out[t] = S
    return (out * y) @ w[pre + "o"].T


# ---------------------------------------------------------------------------------------------------------
def dense_ffn(h, w, pre):
    return (torch.nn.functional.silu(h @ w[pre + "gate"].T) * (h @ w[pre + "up"].T)) @ w[pre + "down"].T


def relu2_expert(x, w, pre):
    return torch.relu(x @ w[pre + "up"].T) ** 2 @ w[pre + "down"].T


def moe_ffn(h, w, pre, mlp, choices=None):
    """Sigmoid router; the chosen experts' scores scale the experts' inputs; a shared expert is added.
    ``choices`` [T, top] overrides the selection (the scores stay the router's)."""
    E, top = mlp["router"]["experts"], mlp["router"]["top"]
    s = torch.sigmoid(h @ w[pre + "router"].T)
    if choices is None:
        # the largest scores, ties to the lower index
        choices = torch.sort(s, dim=-1, descending=True, stable=True).indices[:, :top]
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for e in choices[t].tolist():
            out[t] += relu2_expert(s[t, e] * h[t], w, f"{pre}e{e}.")
    if mlp.get("shared") is not None:
        out = out + relu2_expert(h, w, pre + "shared.")
    return out, choices


# ---------------------------------------------------------------------------------------------------------
def forward(cfg, weights, tokens, dtype=torch.float64, trace=None, choices=None):
    """Logits [T, vocab] of one sequence from its first token on.  ``trace``: a list that receives the residual
    stream after every layer.  ``choices``: {layer: [T, top]} expert selections to use instead of the router's."""
    w = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in weights.items()}
    eps = cfg["norm"]["eps"]
    T = len(tokens)
    positions = torch.arange(T)
    x = embedding(list(tokens), w, cfg, dtype)
    for i, layer in enumerate(cfg["layers"]):
        pre = f"l{i}."
        h = scalar_norm(x, w[pre + "norm1"], eps)
        if layer["type"] == "attention":
            y = sink_attention(h, w, pre + "mix.", layer["mixer"], eps, positions)
        elif layer["type"] == "mlstm":
            y = mlstm(h, w, pre + "mix.", layer["mixer"], eps)
        elif layer["type"] == "rglru":
            y = rglru(h, w, pre + "mix.", layer["mixer"])
        else:
            raise ValueError(layer["type"])
        x = x + scalar_norm(y, w[pre + "norm1b"], eps)
        mlp = layer.get("mlp")
        if mlp is not None:
            h = scalar_norm(x, w[pre + "norm2"], eps)
            if mlp["kind"] == "dense":
                y = dense_ffn(h, w, pre + "mlp.")
            else:
                y, _ = moe_ffn(h, w, pre + "mlp.", mlp, None if choices is None else choices.get(i))
            x = x + scalar_norm(y, w[pre + "norm2b"], eps)
        if trace is not None:
            trace.append(x.clone())
    return scalar_norm(x, w["final.norm"], eps) @ w["head"].T


def tensor_shapes(cfg):
    """name -> shape of every tensor of the design, from the configuration alone."""
    D, Vc = cfg["width"], cfg["vocab"]
    out = {"embed": (Vc, D), "bigram": (cfg["embedding"]["bigram"]["buckets"] + 1, D), "final.norm": (), "head": (Vc, D)}
    for i, layer in enumerate(cfg["layers"]):
        p, mix = f"l{i}.mix.", layer["mixer"]
        out[f"l{i}.norm1"] = out[f"l{i}.norm1b"] = ()
        if layer["type"] == "attention":
            H, K = mix["heads"], mix["dim"]
            G, V = mix.get("kv_heads", H), mix.get("vdim", K)
            out.update({p + "q": (H * K, D), p + "q.b": (H * K,), p + "k": (G * K, D), p + "k.b": (G * K,),
                        p + "v": (G * V, D), p + "v.b": (G * V,), p + "q.norm": (K,), p + "k.norm": (K,), p + "o": (D, H * V)})
        elif layer["type"] == "mlstm":
            H, K, V = mix["heads"], mix["dim"], mix.get("vdim", mix["dim"])
            out.update({p + "q": (H * K, D), p + "k": (H * K, D), p + "v": (H * V, D), p + "g": (H * V, D), p + "o": (D, H * V),
                        p + "norm": (H * V,), p + "i": (H, D), p + "i.b": (H,), p + "f": (H, D), p + "f.b": (H,)})
        else:
            C, B, taps = mix["width"], mix["blocks"], mix["conv"]
            out.update({p + "y": (C, D), p + "y.b": (C,), p + "x": (C, D), p + "x.b": (C,), p + "conv": (C, taps),
                        p + "conv.b": (C,), p + "ra": (B, C // B, C // B), p + "ra.b": (B, C // B), p + "ri": (B, C // B, C // B),
                        p + "ri.b": (B, C // B), p + "lam": (C,), p + "o": (D, C)})
        mlp = layer.get("mlp")
        if mlp is None:
            continue
        out[f"l{i}.norm2"] = out[f"l{i}.norm2b"] = ()
        p = f"l{i}.mlp."
        if mlp["kind"] == "dense":
            out.update({p + "gate": (mlp["ff"], D), p + "up": (mlp["ff"], D), p + "down": (D, mlp["ff"])})
        else:
            F = mlp["expert"]["ff"]
            for e in range(mlp["router"]["experts"]):
                out.update({f"{p}e{e}.up": (F, D), f"{p}e{e}.down": (D, F)})
            out[p + "router"] = (mlp["router"]["experts"], D)
            if mlp.get("shared") is not None:
                out.update({p + "shared.up": (mlp["shared"]["ff"], D), p + "shared.down": (D, mlp["shared"]["ff"])})
    return out


def greedy(cfg, weights, prompt, count):
    """``count`` greedy tokens after ``prompt`` and, for each, the margin between the best and the second logit."""
    seq, margins = list(prompt), []
    for _ in range(count):
        top = torch.topk(forward(cfg, weights, seq)[-1], 2)
        margins.append(float(top.values[0] - top.values[1]))
        seq.append(int(top.indices[0]))
    return seq[len(prompt):], margins
