"""Plain, slow restatement of the Raritar design in float64 torch ops, one function per mechanism.  It shares no code
with the product path: tests build small random checkpoints with `random_model` and compare the framework against this.

Notation: x residual stream [T, W]; a sublayer reads n(x) = g * x / sqrt(mean(x^2) + eps) with ONE number g; the mixer's
input additionally passes u -> u + causal_conv(u) over time; x <- x + m * sublayer(...).  Everything here recomputes a
whole sequence from its first token, so it knows nothing of caches, slots, windows of a cache or batches.
"""
import math

import torch

F64 = torch.float64


def rms(x, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def bigram_rows(tokens, buckets, mul_prev, mul_cur):
    """Row of the bigram table per token: a hash of (previous, current); the table's last row for a first token."""
    rows = [buckets]
    for a, b in zip(tokens[:-1], tokens[1:]):
        rows.append((a * mul_prev + b * mul_cur) % buckets)
    return rows


def time_conv(u, w):
    """u [T, C], w [C, taps]: out_t = sum_j w[:, j] * u_(t - taps + 1 + j), zeros before the start."""
    T, taps = u.shape[0], w.shape[1]
    out = torch.zeros_like(u)
    for t in range(T):
        for j in range(taps):
            s = t - taps + 1 + j
            if s >= 0:
                out[t] += w[:, j] * u[s]
    return out


def rotary_frequencies(dims, base, scaling=None):
    """f_i = base^(-2i/dims); long wavelengths divided by `factor`, short ones kept, a linear blend between."""
    out = []
    for i in range(dims // 2):
        f = base ** (-2.0 * i / dims)
        if scaling:
            fac, lo, hi, orig = (float(scaling[k]) for k in ("factor", "low", "high", "original"))
            wl = 2 * math.pi / f
            if wl < orig / hi:
                pass
            elif wl > orig / lo:
                f = f / fac
            else:
                s = (orig / wl - lo) / (hi - lo)
                f = (1 - s) * f / fac + s * f
        out.append(f)
    return out


def rotate(t, pos, freqs):
    """t [T, heads, dim]: neighbouring coordinates (2i, 2i+1) of the first 2 * len(freqs) are turned by pos * f_i."""
    out = t.clone()
    for i, f in enumerate(freqs):
        a = torch.tensor([p * f for p in pos], dtype=F64)
        c, s = torch.cos(a)[:, None], torch.sin(a)[:, None]
        u, v = t[:, :, 2 * i], t[:, :, 2 * i + 1]
        out[:, :, 2 * i] = u * c - v * s
        out[:, :, 2 * i + 1] = v * c + u * s
    return out


def visible(i, j, window, keep_first):
    return j <= i and (i - j < window or j < keep_first)


def attention_core(q, k, v, scale, softcap, window, keep_first):
    """q [T, H, D], k [T, G, D], v [T, G, V] of ONE sequence from its first token -> [T, H, V]."""
    T, H, _ = q.shape
    G = k.shape[1]
    out = torch.zeros(T, H, v.shape[-1], dtype=F64)
    for i in range(T):
        js = [j for j in range(i + 1) if visible(i, j, window, keep_first)]
        for h in range(H):
            g = h // (H // G)
            s = (k[js, g] @ q[i, h]) * scale
            if softcap:
                s = softcap * torch.tanh(s / softcap)
            p = torch.softmax(s, 0)
            out[i, h] = p @ v[js, g]
    return out


def keys_values(W, p, u, c, eps):
    """The rows an attention layer caches: rotated keys and unit-RMS values."""
    T = u.shape[0]
    G, D, V = c["kv_heads"], c["dim"], c["vdim"]
    rot = c.get("rot") or {}
    freqs = rotary_frequencies(int(rot.get("dims", 0)), float(rot.get("base", 10000.0)), rot.get("scaling")) if rot.get("dims") else []
    k = rotate((u @ W[p + "k"].T).view(T, G, D), range(T), freqs)
    v = rms((u @ W[p + "v"].T).view(T, G, V), eps)
    return k, v


def attention_mixer(W, p, u, c, eps, kv=None):
    """u: the mixer's input [T, W].  `kv`: another layer's (keys, values) when this layer has none of its own."""
    T = u.shape[0]
    H, D = c["heads"], c["dim"]
    rot = c.get("rot") or {}
    freqs = rotary_frequencies(int(rot.get("dims", 0)), float(rot.get("base", 10000.0)), rot.get("scaling")) if rot.get("dims") else []
    q = rotate((u @ W[p + "q"].T).view(T, H, D), range(T), freqs)
    k, v = kv if kv is not None else keys_values(W, p, u, c, eps)
    mask = c.get("mask") or {}
    o = attention_core(q, k, v, float(c["scale"]), float(c.get("softcap") or 0.0), int(mask.get("size", 1 << 40)), int(mask.get("keep_first", 0)))
    return o.reshape(T, -1) @ W[p + "o"].T, (k, v)


def silu(z):
    return z * torch.sigmoid(z)


def gated_ff(W, p, h):
    return (silu(h @ W[p + "gate"].T) * (h @ W[p + "up"].T)) @ W[p + "down"].T


def route(z, correction, top, n_groups, keep_groups):
    """z [E] router logits of ONE token -> (chosen indices, their weights).  Choice by score + correction inside the best
    groups; weights are the plain scores."""
    s = torch.softmax(z, 0)
    choice = s + correction
    E = z.shape[0]
    per = E // n_groups
    best = sorted(range(n_groups), key=lambda g: (-float(choice[g * per:(g + 1) * per].max()), g))[:keep_groups]
    allowed = [e for e in range(E) if e // per in best]
    chosen = sorted(allowed, key=lambda e: (-float(choice[e]), e))[:top]
    return chosen, [s[e] for e in chosen]


def moe_ff(W, p, h, c):
    r = c["router"]
    E, I = int(r["experts"]), int(r.get("identity", 0))
    groups = r.get("groups") or {}
    zs = h @ W[p + "router"].T
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        chosen, ws = route(zs[t], W[p + "correction"], int(r["top"]), int(groups.get("count", 1)), int(groups.get("keep", 1)))
        for e, w in zip(chosen, ws):
            out[t] += w * (h[t] if e >= E else gated_ff(W, f"{p}e{e}.", h[t:t + 1])[0])   # outputs E .. E+I-1 pass h through
    if c.get("shared"):
        out = out + torch.sigmoid(h @ W[p + "shared.sg"].T) * gated_ff(W, p + "shared.", h)
    return out


def forward(cfg, weights, tokens, trace=None):
    """Logits [T, vocab] of one sequence; `trace` (a list) receives the residual stream after every layer."""
    W = {k: (v.to(F64) if v.is_floating_point() else v) for k, v in weights.items()}
    eps, m = float(cfg["norm"]["eps"]), float(cfg.get("residual_mult", 1.0))
    x = W["embed"][tokens]
    bg = (cfg.get("embedding") or {}).get("bigram")
    if bg:
        x = x + W["bigram"][bigram_rows(list(tokens), int(bg["buckets"]), int(bg["mul_prev"]), int(bg["mul_cur"]))]
    taps = int((cfg.get("canon") or {}).get("taps", 0))
    cached = {}
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}."
        u = rms(x, eps) * W[p + "norm1"]
        if taps:
            u = u + time_conv(u, W[p + "canon1"])
        src = layer["mixer"].get("kv_from")
        y, cached[i] = attention_mixer(W, p + "mix.", u, layer["mixer"], eps, cached[src] if src is not None else None)
        x = x + m * y
        if layer.get("mlp"):
            x = x + m * moe_ff(W, p + "mlp.", rms(x, eps) * W[p + "norm2"], layer["mlp"])
        if trace is not None:
            trace.append(x.clone())
    return (rms(x, eps) * W["final.norm"]) @ W["head"].T


def random_model(cfg, seed=0, scale=0.5):
    """Random weights for a configuration (bfloat16, as a checkpoint stores them)."""
    g = torch.Generator().manual_seed(seed)
    Wd, V = int(cfg["width"]), int(cfg["vocab"])

    def mat(o, i, s=None):
        return (torch.randn(o, i, generator=g) * (s if s is not None else scale / math.sqrt(i))).to(torch.bfloat16)

    def num(lo=0.8, hi=1.3):
        return (torch.rand((), generator=g) * (hi - lo) + lo).to(torch.bfloat16)

    W = {"embed": mat(V, Wd, 1.0), "head": mat(V, Wd, 1.5 / math.sqrt(Wd)), "final.norm": num()}
    bg = (cfg.get("embedding") or {}).get("bigram")
    if bg:
        W["bigram"] = mat(int(bg["buckets"]) + 1, Wd, 0.7)
    taps = int((cfg.get("canon") or {}).get("taps", 0))
    for i, layer in enumerate(cfg["layers"]):
        p, c = f"l{i}.", layer["mixer"]
        W[p + "norm1"] = num()
        if taps:
            W[p + "canon1"] = mat(Wd, taps, 0.4)
        H, G, D, Vd = c["heads"], c["kv_heads"], c["dim"], c["vdim"]
        W[p + "mix.q"] = mat(H * D, Wd, 2.0 / math.sqrt(Wd))
        if c.get("kv_from") is None:
            W[p + "mix.k"] = mat(G * D, Wd, 2.0 / math.sqrt(Wd))
            W[p + "mix.v"] = mat(G * Vd, Wd)
        W[p + "mix.o"] = mat(Wd, H * Vd, 1.0 / math.sqrt(H * Vd))
        f = layer.get("mlp")
        if f:
            W[p + "norm2"] = num()
            r = f["router"]
            E, I = int(r["experts"]), int(r.get("identity", 0))
            W[p + "mlp.router"] = mat(E + I, Wd, 3.0 / math.sqrt(Wd))
            W[p + "mlp.correction"] = (torch.randn(E + I, generator=g) * 0.1).to(torch.bfloat16)
            names = [f"e{e}." for e in range(E)] + (["shared."] if f.get("shared") else [])
            for n in names:
                ff = int(f["shared"]["ff"] if n == "shared." else f["expert"]["ff"])
                W[p + "mlp." + n + "gate"] = mat(ff, Wd, 1.5 / math.sqrt(Wd))
                W[p + "mlp." + n + "up"] = mat(ff, Wd, 1.5 / math.sqrt(Wd))
                W[p + "mlp." + n + "down"] = mat(Wd, ff, 1.5 / math.sqrt(ff))
            if f.get("shared"):
                W[p + "mlp.shared.sg"] = mat(1, Wd, 2.0 / math.sqrt(Wd))
    return W


def attn_layer(heads=4, kv_heads=2, dim=16, vdim=8, window=12, keep_first=3, rot_dims=8, scaling=True, softcap=30.0, kv_from=None,
               experts=6, identity=2, top=3, groups=(4, 2), ff=24, shared_ff=16, mlp=True):
    """One layer's configuration entry (small sizes; every key the design reads)."""
    mixer = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "mask": {"size": window, "keep_first": keep_first},
             "rot": {"base": 10000.0, "dims": rot_dims}, "scale": 1.3 / math.sqrt(dim), "softcap": softcap}
    if scaling:
        mixer["rot"]["scaling"] = {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 64}
    if kv_from is not None:
        mixer["kv_from"] = kv_from
    f = None
    if mlp:
        f = {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "identity": identity, "top": top,
                                                            "groups": {"count": groups[0], "keep": groups[1]}}}
        if shared_ff:
            f["shared"] = {"ff": shared_ff}
    return {"type": "attention", "mixer": mixer, "mlp": f}


def make_config(layers, width=40, vocab=61, taps=4, buckets=53, mult=0.6, eps=1e-5):
    cfg = {"architecture": "Raritar", "vocab": vocab, "width": width, "residual_mult": mult, "norm": {"eps": eps}, "layers": layers}
    if taps:
        cfg["canon"] = {"taps": taps}
    if buckets:
        cfg["embedding"] = {"bigram": {"buckets": buckets, "mul_prev": 29, "mul_cur": 5}}
    return cfg
