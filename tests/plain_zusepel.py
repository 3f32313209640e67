"""A plain, slow restatement of the Zusepel decoder, one function per mechanism.

It shares no code with the library: tensors come in as a dict name -> torch
tensor, the configuration as the parsed config.json, and everything runs on the
CPU in one dtype (float64 by default) token by token where the design has a
recurrence.  ``forward`` returns logits for a whole sequence and, optionally,
the residual stream after every layer.

Notation: T tokens, D width, H heads, K key channels per head, V value channels
per head.
"""
from __future__ import annotations

import math

import torch


def rms(x, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def softplus(z):
    return math.log1p(math.exp(z)) if z < 30 else z


def xielu(z, p, q):
    """p, q: the two raw numbers of the activation."""
    ap, aq = softplus(float(p)), 0.5 + softplus(float(q))
    pos = ap * z * z + 0.5 * z
    neg = aq * (torch.expm1(torch.clamp(z, max=0.0)) - z) + 0.5 * z
    return torch.where(z > 0, pos, neg)


def feed_forward(h, w, pre):
    a = xielu(h @ w[pre + "up"].T, w[pre + "act"][0], w[pre + "act"][1])
    return a @ w[pre + "down"].T


# ---------------------------------------------------------------------------------------------------------
def hgrn2(h, w, pre, mix, eps):
    """Gated linear recurrence: S_t = diag(f_t) S_(t-1) + (1 - f_t) v_t^T, o_t = S_t^T q_t."""
    H, K, V = mix["heads"], mix["dim"], mix["vdim"]
    T = h.shape[0]
    q = torch.nn.functional.silu(h @ w[pre + "q"].T).view(T, H, K)
    v = (h @ w[pre + "v"].T).view(T, H, V)
    lower = w[pre + "lower"].view(H, K)
    f = lower + (1 - lower) * torch.sigmoid(h @ w[pre + "f"].T + w[pre + "f.b"]).view(T, H, K)
    S = torch.zeros(H, K, V, dtype=h.dtype)
    out = torch.zeros(T, H, V, dtype=h.dtype)
    for t in range(T):
        S = f[t][:, :, None] * S + (1 - f[t])[:, :, None] * v[t][:, None, :]
        out[t] = torch.einsum("hkv,hk->hv", S, q[t])
    out = rms(out, eps) * w[pre + "norm"]
    return out.reshape(T, H * V) @ w[pre + "o"].T


def wkv(h, w, pre, mix, eps):
    """Token-shifted projections, a decay per key channel computed from the input, an extra weight u on the token being read."""
    H, K = mix["heads"], mix["dim"]
    T, D = h.shape
    prev = torch.cat([torch.zeros(1, D, dtype=h.dtype), h[:-1]], 0)
    mixed = {s: h + (prev - h) * w[pre + "mu." + s] for s in "rkvgw"}
    r = (mixed["r"] @ w[pre + "r"].T).view(T, H, K)
    k = (mixed["k"] @ w[pre + "k"].T).view(T, H, K)
    v = (mixed["v"] @ w[pre + "v"].T).view(T, H, K)
    gate = torch.nn.functional.silu(mixed["g"] @ w[pre + "g"].T)
    decay = torch.exp(-torch.exp(torch.tanh(mixed["w"] @ w[pre + "w1"].T) @ w[pre + "w2"].T + w[pre + "w0"])).view(T, H, K)
    u = w[pre + "u"].view(H, K)
    S = torch.zeros(H, K, K, dtype=h.dtype)
    out = torch.zeros(T, H, K, dtype=h.dtype)
    for t in range(T):
        kv = k[t][:, :, None] * v[t][:, None, :]
        out[t] = torch.einsum("hkv,hk->hv", S + u[:, :, None] * kv, r[t])
        S = decay[t][:, :, None] * S + kv
    out = rms(out, eps).reshape(T, H * K) * w[pre + "norm"] * gate
    return out @ w[pre + "o"].T


def rotary_tables(rot, positions, dtype):
    """cos, sin [T, dims/2] with the interpolation of the slow frequencies and the magnitude factor."""
    dims, base = rot["dims"], rot["base"]
    i = torch.arange(dims // 2, dtype=torch.float64)
    f = base ** (-2 * i / dims)
    mag = 1.0
    sc = rot.get("scaling")
    if sc:
        def corr(turns):
            return dims * math.log(sc["original"] / (2 * math.pi * turns)) / (2 * math.log(base))
        lo = max(math.floor(corr(sc["fast"])), 0)
        hi = min(math.ceil(corr(sc["slow"])), dims - 1)
        ramp = torch.clamp((i - lo) / max(hi - lo, 0.001), 0, 1)
        f = f / sc["factor"] * ramp + f * (1 - ramp)
        mag = 0.1 * math.log(sc["factor"]) + 1
    ang = positions.to(torch.float64)[:, None] * f.to(torch.float32).to(torch.float64)[None, :]
    return (torch.cos(ang) * mag).to(dtype), (torch.sin(ang) * mag).to(dtype)


def rotate(x, cos, sin, dims):
    """x [T, ..., R]; the first ``dims`` of R are rotated in pairs (i, i + dims/2)."""
    half = dims // 2
    a, b, rest = x[..., :half], x[..., half:dims], x[..., dims:]
    while cos.dim() < a.dim():
        cos, sin = cos.unsqueeze(1), sin.unsqueeze(1)
    return torch.cat([a * cos - b * sin, b * cos + a * sin, rest], -1)


def latent_kv(h, w, pre, mix, eps, positions):
    """What the layer caches: the normed latent [T, rank] and the rotated shared key part [T, rot_dim]."""
    R = mix["kv_rank"]
    d = h @ w[pre + "dkv"].T
    c = rms(d[:, :R], eps) * w[pre + "dkv.norm"]
    cos, sin = rotary_tables(mix["rot"], positions, h.dtype)
    return c, rotate(d[:, R:], cos, sin, mix["rot"]["dims"])


def latent_attention(h, w, pre, mix, eps, positions, c, kr):
    """c, kr: latent and rotated key part of every position (this layer's own or another layer's)."""
    H, K, R, V = mix["heads"], mix["dim"], mix["rot_dim"], mix["vdim"]
    T = h.shape[0]
    cq = rms(h @ w[pre + "dq"].T, eps) * w[pre + "dq.norm"]
    q = (cq @ w[pre + "uq"].T).view(T, H, K + R)
    cos, sin = rotary_tables(mix["rot"], positions, h.dtype)
    q_rot = rotate(q[..., K:], cos, sin, mix["rot"]["dims"])
    k_nope = (c @ w[pre + "uk"].T).view(T, H, K)
    val = (c @ w[pre + "uv"].T).view(T, H, V)
    score = (torch.einsum("thk,shk->hts", q[..., :K], k_nope) + torch.einsum("thr,sr->hts", q_rot, kr)) * mix["scale"]
    i = positions[:, None]
    j = positions[None, :]
    seen = (j <= i)
    if mix.get("mask"):
        seen = seen & (i - j < mix["mask"]["size"])
    score = score.masked_fill(~seen[None], float("-inf"))
    out = torch.einsum("hts,shv->thv", torch.softmax(score, -1), val)
    return out.reshape(T, H * V) @ w[pre + "o"].T


# ---------------------------------------------------------------------------------------------------------
def forward(cfg, weights, tokens, dtype=torch.float64, layers_out=None):
    """Logits [T, vocab] of one sequence from its first token on."""
    w = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in weights.items()}
    eps, m = cfg["norm"]["eps"], cfg["residual_mult"]
    tokens = torch.as_tensor(tokens, dtype=torch.long)
    positions = torch.arange(tokens.shape[0])
    x = w["embed"][tokens]
    streams = [x]
    kept = {}
    for i, layer in enumerate(cfg["layers"]):
        pre, mix = f"l{i}.mix.", layer["mixer"]
        h = rms(x, eps) * w[f"l{i}.norm1"]
        if layer["type"] == "hgrn2":
            y = hgrn2(h, w, pre, mix, eps)
        elif layer["type"] == "wkv":
            y = wkv(h, w, pre, mix, eps)
        elif layer["type"] == "latent_attention":
            if mix.get("kv_from") is None:
                kept[i] = latent_kv(h, w, pre, mix, eps, positions)
            c, kr = kept[i if mix.get("kv_from") is None else mix["kv_from"]]
            y = latent_attention(h, w, pre, mix, eps, positions, c, kr)
        else:
            raise ValueError(layer["type"])
        x = x + m * (y * w[f"l{i}.ls1"])
        if layer.get("mlp") is not None:
            h = rms(x, eps) * w[f"l{i}.norm2"]
            x = x + m * (feed_forward(h, w, f"l{i}.mlp.") * w[f"l{i}.ls2"])
        streams.append(x)
        x = sum(w[f"l{i}.dwa"][j] * streams[j] for j in range(i + 2))
        if layers_out is not None:
            layers_out.append(x.clone())
    h = rms(x, eps) * w["final.norm"]
    return h @ w["head"].T


# ---------------------------------------------------------------------------------------------------------
# tensors of a model, listed from the design (not from the library), and random values that keep every
# mechanism alive: decays near one and near zero, bounds inside (0, 1), scales away from one
def tensor_shapes(cfg, decay_rank=16):
    D, shapes = cfg["width"], {}
    shapes["embed"] = (cfg["vocab"], D)
    shapes["head"] = (cfg["vocab"], D)
    shapes["final.norm"] = (D,)
    for i, layer in enumerate(cfg["layers"]):
        p, mix = f"l{i}.", layer["mixer"]
        shapes[p + "norm1"] = (D,)
        shapes[p + "ls1"] = (D,)
        shapes[p + "dwa"] = (i + 2,)
        H = mix["heads"]
        if layer["type"] == "hgrn2":
            K, V = mix["dim"], mix["vdim"]
            shapes.update({p + "mix.q": (H * K, D), p + "mix.f": (H * K, D), p + "mix.f.b": (H * K,), p + "mix.lower": (H * K,),
                           p + "mix.v": (H * V, D), p + "mix.norm": (V,), p + "mix.o": (D, H * V)})
        elif layer["type"] == "wkv":
            K = mix["dim"]
            for s in "rkvgw":
                shapes[p + "mix.mu." + s] = (D,)
            for s in "rkvg":
                shapes[p + "mix." + s] = (H * K, D)
            shapes.update({p + "mix.w1": (decay_rank, D), p + "mix.w2": (H * K, decay_rank), p + "mix.w0": (H * K,),
                           p + "mix.u": (H, K), p + "mix.norm": (H * K,), p + "mix.o": (D, H * K)})
        else:
            K, R, V = mix["dim"], mix["rot_dim"], mix["vdim"]
            shapes.update({p + "mix.dq": (mix["q_rank"], D), p + "mix.dq.norm": (mix["q_rank"],),
                           p + "mix.uq": (H * (K + R), mix["q_rank"]), p + "mix.uk": (H * K, mix["kv_rank"]),
                           p + "mix.uv": (H * V, mix["kv_rank"]), p + "mix.o": (D, H * V)})
            if mix.get("kv_from") is None:
                shapes.update({p + "mix.dkv": (mix["kv_rank"] + R, D), p + "mix.dkv.norm": (mix["kv_rank"],)})
        if layer.get("mlp") is not None:
            ff = layer["mlp"]["ff"]
            shapes.update({p + "norm2": (D,), p + "ls2": (D,), p + "mlp.up": (ff, D), p + "mlp.down": (D, ff),
                           p + "mlp.act": (2,)})
    return shapes


def random_weights(cfg, seed, decay_rank=16, gain=1.0):
    """name -> bfloat16 tensor (what a model folder stores)."""
    g = torch.Generator().manual_seed(seed)
    rn = lambda *s: torch.randn(*s, generator=g)
    ru = lambda *s: torch.rand(*s, generator=g)
    out = {}
    for name, shape in tensor_shapes(cfg, decay_rank).items():
        leaf = name.split(".", 1)[1] if name.startswith("l") and name[1].isdigit() else name
        if len(shape) == 2 and leaf != "mix.u":
            t = rn(*shape) * (gain / math.sqrt(shape[1]))
            if name == "embed":
                t = rn(*shape)
        elif leaf in ("norm1", "norm2", "mix.norm", "mix.dq.norm", "mix.dkv.norm") or name == "final.norm":
            t = 1 + 0.2 * rn(*shape)
        elif leaf in ("ls1", "ls2"):
            t = 0.4 + 0.8 * ru(*shape)
        elif leaf == "dwa":
            t = (0.3 + ru(*shape))
            t = t / t.sum() * (1 + 0.1 * rn(1))
        elif leaf.startswith("mix.mu."):
            t = ru(*shape)
        elif leaf == "mix.w0":
            t = rn(*shape) * 1.5 - 1.5            # decays from about 0.2 to nearly 1
        elif leaf == "mix.u":
            t = 0.5 * rn(*shape)
        elif leaf == "mix.lower":
            t = 0.95 * ru(*shape)
        elif leaf == "mix.f.b":
            t = rn(*shape)
        elif leaf == "mlp.act":
            t = 0.7 * rn(*shape)
        else:
            raise ValueError(name)
        out[name] = t.to(torch.bfloat16)
    return out


def greedy(cfg, weights, prompt, n_new, dtype=torch.float64):
    """Greedy continuation by running the whole sequence anew for every token; returns (tokens, the margin
    between the best and the second logit at every choice)."""
    toks, margins = list(prompt), []
    for _ in range(n_new):
        top = torch.topk(forward(cfg, weights, toks, dtype)[-1], 2)
        toks.append(int(top.indices[0]))
        margins.append(float(top.values[0] - top.values[1]))
    return toks[len(prompt):], margins
