"""Plain, slow restatement of the Mutolix design in float64 torch ops, one function per mechanism.  It shares no code
with the product path: tests build small random checkpoints with `random_model` and compare the framework against this.

Notation: x residual stream [T, W]; h = rms(x) * w the input of a sublayer; every sublayer result y goes through
x + ls * w_b * rms(y * sigmoid(W_rg h + b_rg)).
"""
import math

import torch

F64 = torch.float64


def rms(x, eps, w=None):
    y = x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)
    return y if w is None else y * w


def softplus(z):
    return math.log1p(math.exp(z))


def xielu(z, a_pos, a_neg):
    """z > 0: softplus(a_pos) z^2 + z/2; z <= 0: (1/2 + softplus(a_neg)) (e^z - 1 - z) + z/2."""
    cp, cn = softplus(a_pos), 0.5 + softplus(a_neg)
    neg = torch.clamp(z, max=0.0)
    return torch.where(z > 0, cp * z * z + z / 2, cn * (torch.exp(neg) - 1 - neg) + z / 2)


def mlstm_gates(h, w_i, b_i, w_f, b_f, cap):
    i = cap * torch.tanh((h @ w_i.T + b_i) / cap)
    f = torch.nn.functional.logsigmoid(cap * torch.tanh((h @ w_f.T + b_f) / cap))
    return i, f


def mlstm_recurrence(q, k, v, ig, fg, state=None):
    """q, k [T, H, D] (q already scaled), v [T, H, V], gates [T, H].  Returns (o [T, H, V], state); state = (S, n, m)."""
    T, H, D = q.shape
    V = v.shape[-1]
    if state is None:
        S, n, m = torch.zeros(H, D, V, dtype=q.dtype), torch.zeros(H, D, dtype=q.dtype), torch.zeros(H, dtype=q.dtype)
    else:
        S, n, m = (t.clone() for t in state)
    out = torch.zeros(T, H, V, dtype=q.dtype)
    for t in range(T):
        m_new = torch.maximum(fg[t] + m, ig[t])
        a, b = torch.exp(fg[t] + m - m_new), torch.exp(ig[t] - m_new)
        S = a[:, None, None] * S + b[:, None, None] * k[t][:, :, None] * v[t][:, None, :]
        n = a[:, None] * n + b[:, None] * k[t]
        m = m_new
        den = torch.maximum((n * q[t]).sum(-1).abs(), torch.exp(-m)) + 1e-6
        out[t] = torch.einsum("hdv,hd->hv", S, q[t]) / den[:, None]
    return out, (S, n, m)


def mlstm_mixer(W, p, h, c, eps, state=None):
    H, D, V = c["heads"], c["dim"], c["vdim"]
    T = h.shape[0]
    q = (h @ W[p + "q"].T * D ** -0.5).view(T, H, D)
    k = (h @ W[p + "k"].T).view(T, H, D)
    v = (h @ W[p + "v"].T).view(T, H, V)
    ig, fg = mlstm_gates(h, W[p + "i"], W[p + "i.b"], W[p + "f"], W[p + "f.b"], c["gate_cap"])
    o, state = mlstm_recurrence(q, k, v, ig, fg, state)
    o = rms(o, eps).reshape(T, H * V) * W[p + "norm"] * torch.sigmoid(h @ W[p + "g"].T)
    return o @ W[p + "o"].T, state


def sink_attention(q, k, v, pos_q, pos_k, scale, r1=None, r2=None, sink=True):
    """q [Tq, H, D], k [Tk, G, D], v [Tk, G, V]; positions as integer tensors.  Causal: key j is seen when pos_k <= pos_q.
    p_j = exp(s_j) / (sink + sum exp(s_j)) with sink = 1 (a score of 0 that carries no value) or 0."""
    Tq, H, _ = q.shape
    G = k.shape[1]
    out = torch.zeros(Tq, H, v.shape[-1], dtype=q.dtype)
    dist = (pos_q[:, None] - pos_k[None, :]).clamp(min=0).to(q.dtype)
    hidden = pos_k[None, :] > pos_q[:, None]
    for hh in range(H):
        g = hh // (H // G)
        s = q[:, hh] @ k[:, g].T * scale
        if r1 is not None:
            s = s - r1[hh] * torch.log(1 + r2[hh] * dist)
        s = s.masked_fill(hidden, -float("inf"))
        mx = s.max(-1, keepdim=True).values.clamp(min=0.0)
        e = torch.exp(s - mx)
        den = e.sum(-1, keepdim=True) + (torch.exp(-mx) if sink else 0.0)
        out[:, hh] = (e / den) @ v[:, g]
    return out


def attention_qkv(W, p, h, c, eps, pos, v_first=None):
    """The prepared q, k and (mixed) v of the tokens at positions `pos`."""
    H, G, D, V = c["heads"], c["kv_heads"], c["dim"], c["vdim"]
    T = h.shape[0]
    q = rms(h @ W[p + "q"].T + W[p + "q.b"], eps, W[p + "q.norm"])
    k = rms(h @ W[p + "k"].T + W[p + "k.b"], eps, W[p + "k.norm"])
    v = h @ W[p + "v"].T + W[p + "v.b"]
    qt = c.get("q_temp")
    if qt:
        q = q * (1 + qt["coef"] * torch.log(torch.floor((pos + 1) / qt["every"]).to(q.dtype) + 1))[:, None]
    if v_first is not None:
        lam = W[p + "vmix"]
        v = (1 - lam) * v + lam * v_first
    return q.view(T, H, D), k.view(T, G, D), v.view(T, G, V)


def forward(cfg, W, tokens, layers_out=None):
    """Logits [T, vocab] of one sequence run whole."""
    eps = cfg["norm"]["eps"]
    tokens = torch.as_tensor(tokens)
    T = tokens.shape[0]
    pos = torch.arange(T)
    x = W["embed"][tokens] * cfg["embedding"]["scale"]
    v_first = None
    for i, L in enumerate(cfg["layers"]):
        p, c = f"l{i}.", L["mixer"]
        h = rms(x, eps, W[p + "norm1"])
        if L["type"] == "mlstm":
            y, _ = mlstm_mixer(W, p + "mix.", h, c, eps)
        else:
            mix = v_first if c.get("v_mix") else None
            q, k, v = attention_qkv(W, p + "mix.", h, c, eps, pos, mix)
            if c.get("v_mix") and v_first is None:
                v_first = v.reshape(T, -1)
            o = sink_attention(q, k, v, pos, pos, c["scale"], W[p + "mix.r1"], W[p + "mix.r2"])
            y = o.reshape(T, -1) @ W[p + "mix.o"].T
        y = y * torch.sigmoid(h @ W[p + "rg1"].T + W[p + "rg1.b"])
        x = x + rms(y, eps, W[p + "norm1b"]) * W[p + "ls1"]
        if L["mlp"] is not None:
            h = rms(x, eps, W[p + "norm2"])
            a = W[p + "mlp.act"]
            y = xielu(h @ W[p + "mlp.up"].T, float(a[0]), float(a[1])) @ W[p + "mlp.down"].T
            y = y * torch.sigmoid(h @ W[p + "rg2"].T + W[p + "rg2.b"])
            x = x + rms(y, eps, W[p + "norm2b"]) * W[p + "ls2"]
        if layers_out is not None:
            layers_out.append(x.clone())
    return rms(x, eps, W["final.norm"]) @ W["head"].T


def greedy(cfg, W, prompt, n_new):
    toks = list(prompt)
    for _ in range(n_new):
        toks.append(int(torch.argmax(forward(cfg, W, toks)[-1])))
    return toks[len(prompt):]


# ---- small random checkpoints ------------------------------------------------------------------------------------
def mlstm_layer(heads=2, dim=8, vdim=16, gate_cap=10.0, ff=None):
    return {"type": "mlstm", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "gate_cap": gate_cap},
            "mlp": {"kind": "dense", "ff": ff} if ff else None}


def attn_layer(heads=4, kv_heads=2, dim=16, vdim=8, scale=None, coef=0.25, every=8, v_mix=True, ff=48):
    mixer = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale if scale is not None else dim ** -0.5,
             "v_mix": v_mix}
    if every:
        mixer["q_temp"] = {"coef": coef, "every": every}
    return {"type": "attention", "mixer": mixer, "mlp": {"kind": "dense", "ff": ff} if ff else None}


def random_model(layers, width=40, vocab=61, seed=0, emb_scale=0.7, eps=1e-5, bf16_values=True):
    """(config dict, float64 weights).  With `bf16_values` every weight is exactly representable in bfloat16, so that a
    checkpoint written in bfloat16 holds the same numbers the oracle uses."""
    g = torch.Generator().manual_seed(seed)
    cfg = {"architecture": "Mutolix", "vocab": vocab, "width": width, "embedding": {"scale": emb_scale}, "norm": {"eps": eps},
           "layers": layers}
    W = {}

    def rnd(*shape, std=1.0, mean=0.0):
        t = torch.randn(tuple(shape), generator=g, dtype=F64) * std + mean
        return t.to(torch.bfloat16).to(F64) if bf16_values else t

    lin = lambda o, i: rnd(o, i, std=i ** -0.5)
    W["embed"] = rnd(vocab, width)
    for i, L in enumerate(layers):
        p, c = f"l{i}.", L["mixer"]
        for n in ("norm1", "norm1b"):
            W[p + n] = rnd(width, std=0.1, mean=1.0)
        W[p + "ls1"] = rnd(width, std=0.2, mean=0.8)
        W[p + "rg1"], W[p + "rg1.b"] = lin(width, width), rnd(width, std=0.5)
        if L["type"] == "mlstm":
            H, D, V = c["heads"], c["dim"], c["vdim"]
            W[p + "mix.q"], W[p + "mix.k"] = lin(H * D, width), lin(H * D, width)
            W[p + "mix.v"], W[p + "mix.g"] = lin(H * V, width), lin(H * V, width)
            W[p + "mix.o"], W[p + "mix.norm"] = lin(width, H * V), rnd(H * V, std=0.1, mean=1.0)
            W[p + "mix.i"], W[p + "mix.i.b"] = lin(H, width) * 2, rnd(H, std=1.0)
            W[p + "mix.f"], W[p + "mix.f.b"] = lin(H, width) * 2, rnd(H, std=1.0, mean=3.0)
        else:
            H, G, D, V = c["heads"], c["kv_heads"], c["dim"], c["vdim"]
            for n, rows in (("q", H * D), ("k", G * D), ("v", G * V)):
                W[p + "mix." + n], W[p + "mix." + n + ".b"] = lin(rows, width), rnd(rows, std=0.3)
            W[p + "mix.q.norm"], W[p + "mix.k.norm"] = rnd(H * D, std=0.2, mean=1.5), rnd(G * D, std=0.2, mean=1.5)
            W[p + "mix.vmix"] = rnd(std=0.1, mean=0.4)
            W[p + "mix.r1"], W[p + "mix.r2"] = rnd(H, std=0.1, mean=0.5).abs(), rnd(H, std=0.2, mean=0.6).abs()
            W[p + "mix.o"] = lin(width, H * V)
        if L["mlp"] is not None:
            ff = L["mlp"]["ff"]
            for n in ("norm2", "norm2b"):
                W[p + n] = rnd(width, std=0.1, mean=1.0)
            W[p + "ls2"] = rnd(width, std=0.2, mean=0.8)
            W[p + "rg2"], W[p + "rg2.b"] = lin(width, width), rnd(width, std=0.5)
            W[p + "mlp.up"], W[p + "mlp.down"], W[p + "mlp.act"] = lin(ff, width), lin(width, ff), rnd(2, std=0.5)
    W["final.norm"], W["head"] = rnd(width, std=0.1, mean=1.0), lin(vocab, width)
    return cfg, W
