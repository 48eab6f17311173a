"""Raritar: a decoder-only model of attention layers with a sliding window, shared key/value rows and a mixture-of-experts
feed-forward.

    embedding     token row + a row of a hashed (previous token, token) table                     (`pcs_embed_bigram`)
    every layer   x += m * mixer(u + conv(u)),  u = g1 * rms(x)      one norm number per sublayer, a short causal convolution
                  x += m * ff(g2 * rms(x))                            over time on the mixer's input  (`pcs_norm_conv`)
    attention     grouped heads; a leading part of every query / key head is rotated by position in neighbouring pairs with a
                  frequency table that is rescaled for long wavelengths; values are cached at unit RMS per head
                  (`pcs_rope_kv_prep`); the scaled score is capped by cap * tanh(s / cap); a query sees its window and the
                  first tokens of the sequence (`pcs_attn`).  A layer with `kv_from` appends no rows: it reads the rows of
                  the layer it names with its own queries and mask.
    feed-forward  router in 32-bit: softmax scores, choice by score + correction inside the best groups of neighbouring
                  outputs, weights = the plain scores; the last outputs are pass-through experts that hand on the input; a
                  shared expert, gated by one sigmoid per token, is added  (`pcs_moe_route`, `pcs_moe_rows_*` /
                  `pcs_moe_gemm`, `pcs_moe_combine`).

The K/V rows stay in the slot pool for the whole sequence (a window only bounds what a query reads, so the work per token is
bounded while any position can still be continued from).  The previous token and the convolution's last inputs are part of
a sequence's state (`SeqState.last_token`, the pool's double-buffered tails).  Sizes, the order of layers and every constant
come from config.json; tensors are named l<i>.norm1, l<i>.canon1, l<i>.mix.q, l<i>.mlp.e<j>.gate, ... in the checkpoint.
"""
from __future__ import annotations

import json
import math
import os
from typing import Dict, List, Optional

import torch

from .. import _native_seq as nsq
from .. import weights as wio
from ._seqbase import SlotPoolCausalLM
from ._state import ConvTailSpec, KVSpec


def scaled_frequencies(dims: int, base: float, scaling: Optional[dict]) -> List[float]:
    """Angular frequencies base^(-2i/dims) of the rotated pairs.  With `scaling` {factor, low, high, original}: a wavelength
    below original/high keeps its frequency, one above original/low has it divided by factor, and between the two the
    frequency is blended linearly in original/wavelength."""
    out = []
    for i in range(dims // 2):
        f = float(base) ** (-2.0 * i / dims)
        if scaling:
            factor, low, high, orig = (float(scaling[k]) for k in ("factor", "low", "high", "original"))
            wavelength = 2.0 * math.pi / f
            if wavelength > orig / low:
                f = f / factor
            elif wavelength >= orig / high:
                s = (orig / wavelength - low) / (high - low)
                f = (1.0 - s) * f / factor + s * f
        out.append(f)
    return out


class RaritarConfig:
    """config.json of the design: {"architecture", "vocab", "width", "residual_mult", "norm": {"eps"}, "canon": {"taps"},
    "embedding": {"bigram": {"buckets", "mul_prev", "mul_cur"}}, "layers": [{"type": "attention", "mixer": {...}, "mlp": {...} | null}]}."""

    def __init__(self, d: dict):
        self.raw = d
        self.architecture = d.get("architecture", "Raritar")
        self.vocab_size = int(d["vocab"])
        self.width = int(d["width"])
        self.eps = float(d["norm"]["eps"])
        self.residual_mult = float(d.get("residual_mult", 1.0))
        self.taps = int((d.get("canon") or {}).get("taps", 0))
        self.bigram = (d.get("embedding") or {}).get("bigram")
        self.layers = []
        for i, layer in enumerate(d["layers"]):
            if layer["type"] != "attention":
                raise ValueError(f"layer {i}: unknown mixer type {layer['type']!r}")
            mlp = layer.get("mlp")
            if mlp is not None and mlp.get("kind", "moe") != "moe":
                raise ValueError(f"layer {i}: unknown feed-forward kind {mlp.get('kind')!r}")
            self.layers.append({"type": layer["type"], "mixer": dict(layer["mixer"]), "mlp": dict(mlp) if mlp is not None else None})
        self.num_hidden_layers = len(self.layers)

    @classmethod
    def from_dir(cls, path: str) -> "RaritarConfig":
        with open(os.path.join(path, "config.json")) as fh:
            return cls(json.load(fh))


class RaritarForCausalLM(SlotPoolCausalLM):
    def __init__(self, config: RaritarConfig, tensors: Dict[str, torch.Tensor], device="cuda", dtype=torch.bfloat16,
                 max_tokens: Optional[int] = None):
        super().__init__()
        if dtype not in (torch.bfloat16, torch.float32):
            raise ValueError("Raritar computes in bfloat16 or float32")
        self.config, self.compute_dtype = config, dtype
        self.vocab_size, self.width, self.eps, self.mult = config.vocab_size, config.width, config.eps, config.residual_mult
        dev = torch.device(device)

        def get(name):
            t = tensors.get(name)
            if t is None:
                raise KeyError(f"the checkpoint has no tensor {name!r}")
            return t.to(dev, dtype).contiguous()

        self.embed, self.head = get("embed"), get("head")
        self.final_norm = get("final.norm").reshape(1).expand(self.width).contiguous()   # one number, spread over the channels
        self.pair_table = get("bigram") if config.bigram else None
        if config.bigram and self.pair_table.shape[0] != int(config.bigram["buckets"]) + 1:
            raise ValueError("the bigram table must have buckets + 1 rows")
        self.blocks: List[dict] = []
        for i, layer in enumerate(config.layers):
            p, m = f"l{i}.", layer["mixer"]
            H, D, V = int(m["heads"]), int(m["dim"]), int(m["vdim"])
            G = int(m.get("kv_heads", H))
            if H % G:
                raise ValueError(f"layer {i}: {H} heads do not divide into {G} key/value heads")
            rot = m.get("rot") or {}
            rd = int(rot.get("dims", 0))
            mask = m.get("mask") or {}
            src = m.get("kv_from")
            blk = {"heads": H, "kv_heads": G, "dim": D, "vdim": V, "rot_dims": rd,
                   "freqs": torch.tensor(scaled_frequencies(rd, float(rot.get("base", 10000.0)), rot.get("scaling")), dtype=torch.float64,
                                         device=dev) if rd else None,
                   "scale": float(m.get("scale", D ** -0.5)), "softcap": float(m.get("softcap") or 0.0),
                   "window": int(mask.get("size", 0)), "keep_first": int(mask.get("keep_first", 0)),
                   "norm1": get(p + "norm1").reshape(1), "canon": get(p + "canon1").t().contiguous() if config.taps else None,   # [taps, width] for the kernel
                   "w_o": get(p + "mix.o")}
            if src is None:
                blk.update(kv_src=i, w_in=torch.cat([get(p + "mix.q"), get(p + "mix.k"), get(p + "mix.v")], 0).contiguous(),
                           offs=(0, H * D, (H + G) * D), kv=KVSpec(G, D, V))
            else:
                src = int(src)
                if not 0 <= src < i or config.layers[src]["mixer"].get("kv_from") is not None:
                    raise ValueError(f"layer {i}: kv_from must name an earlier layer that has keys and values of its own")
                f = config.layers[src]["mixer"]
                if (int(f.get("kv_heads", f["heads"])), int(f["dim"]), int(f["vdim"])) != (G, D, V):
                    raise ValueError(f"layer {i}: the rows of layer {src} do not have this layer's shape")
                blk.update(kv_src=src, w_in=get(p + "mix.q"), offs=(0, None, None), kv=None)
            f = layer["mlp"]
            blk["mlp"] = f is not None
            if f is not None:
                r = f["router"]
                E, I = int(r["experts"]), int(r.get("identity", 0))
                groups = r.get("groups") or {}
                blk.update(norm2=get(p + "norm2").reshape(1), n_experts=E, top=int(r["top"]), n_groups=int(groups.get("count", 1)),
                           keep_groups=int(groups.get("keep", groups.get("count", 1))), w_router=get(p + "mlp.router"),
                           correction=tensors[p + "mlp.correction"].to(dev, torch.float32).contiguous() if p + "mlp.correction" in tensors else None)
                if blk["w_router"].shape[0] != E + I:
                    raise ValueError(f"layer {i}: the router has {blk['w_router'].shape[0]} outputs, not {E} experts + {I} pass-through")
                if E:
                    blk["w_gu"] = torch.stack([torch.cat([get(f"{p}mlp.e{e}.gate"), get(f"{p}mlp.e{e}.up")], 0) for e in range(E)]).contiguous()
                    blk["w_down"] = torch.stack([get(f"{p}mlp.e{e}.down") for e in range(E)]).contiguous()
                blk["shared"] = bool(f.get("shared"))
                if blk["shared"]:
                    blk["ws_gu"] = torch.cat([get(p + "mlp.shared.gate"), get(p + "mlp.shared.up")], 0).contiguous()
                    blk["ws_down"] = get(p + "mlp.shared.down")
                    blk["w_sg"] = get(p + "mlp.shared.sg").reshape(-1) if p + "mlp.shared.sg" in tensors else None
            self.blocks.append(blk)
        # bfloat16 products accumulate in 32-bit all the way (no reduced-precision split-K sums); float32 stays true float32
        torch.backends.cuda.matmul.allow_bf16_reduced_precision_reduction = False
        torch.backends.cuda.matmul.allow_tf32 = False
        torch.backends.cudnn.allow_tf32 = False
        self.attn_impl = 0
        self.moe_grouped = None   # None: by size; False / "library" / "own" force the row kernels or one of the grouped products
        self._init_runtime(dev, max_tokens)

    def state_specs(self):
        tail = ConvTailSpec(self.config.taps, self.width) if self.config.taps > 1 else None
        return [tuple(s for s in (b["kv"], tail) if s is not None) or None for b in self.blocks]

    @classmethod
    def from_pretrained(cls, path: str, device="cuda", dtype=torch.bfloat16, max_tokens: Optional[int] = None, **_):
        """`path`: a folder with config.json and model.safetensors."""
        cfg = RaritarConfig.from_dir(path)
        tensors = wio.load_file(os.path.join(path, "model.safetensors"), device=device)
        return cls(cfg, tensors, device=device, dtype=dtype, max_tokens=max_tokens)

    # ---- the layers over one batch ------------------------------------------------------------------------------
    def _mixer_input(self, x, h, i, batch):
        blk = self.blocks[i]
        nsq.norm_conv(x, blk["norm1"], self.eps, h, conv_w=blk["canon"], tail=self.pool.layers[i].get("tail"), batch=batch)

    def _layers(self, ids: torch.Tensor, batch, rows: Optional[torch.Tensor]) -> torch.Tensor:
        T, W, dt, dev, eps, m = ids.shape[0], self.width, self.compute_dtype, self._device, self.eps, self.mult
        x = torch.empty(T, W, dtype=torch.float32, device=dev)     # the residual stream, 32-bit, updated in place
        h = torch.empty(T, W, dtype=dt, device=dev)                # the normed input of the next sublayer
        if self.pair_table is not None:
            bg = self.config.bigram
            nsq.embed_bigram(self.embed, self.pair_table, ids, batch.prev_ids, x, int(bg["buckets"]), int(bg["mul_prev"]), int(bg["mul_cur"]))
        else:
            nsq.embed(self.embed, ids, x, 1.0)
        self._mixer_input(x, h, 0, batch)
        for i, blk in enumerate(self.blocks):
            H, G, D, V = blk["heads"], blk["kv_heads"], blk["dim"], blk["vdim"]
            st = self.pool.layers[blk["kv_src"]]
            proj = nsq.linear(h, blk["w_in"])
            q = torch.empty(T, H * D, dtype=dt, device=dev)
            own = blk["kv"] is not None
            nsq.rope_kv_prep(proj, blk["offs"], H, G, D, V, blk["freqs"], blk["rot_dims"], True, True, eps, q,
                             st["k"] if own else None, st["v"] if own else None, batch)
            mixed = torch.empty(T, H * V, dtype=dt, device=dev)
            # few tokens (decoding): the visible keys are split over more blocks; the bound is the window or the pool's
            # capacity, so that a replayed graph stays valid while the sequences grow
            seen = min(self.pool.cap, blk["window"] + blk["keep_first"]) if blk["window"] > 0 else self.pool.cap
            ws = nsq.attn_workspace(T, H, V, dev) if T <= 16 else None
            nsq.attention(q, st["k"], st["v"], mixed, H, blk["scale"], None, None, False, batch, impl=self.attn_impl, max_keys=seen,
                          workspace=ws, softcap=blk["softcap"], window=blk["window"], keep_first=blk["keep_first"])
            y = nsq.linear(mixed, blk["w_o"])
            if blk["mlp"]:
                nsq.norm_conv(x, blk["norm2"], eps, h, y=y, y_mult=m)       # x += m * y;  h = g2 * rms(x)
                idx, wgt, sg = nsq.moe_route(h, blk["w_router"], blk["correction"], blk.get("w_sg") if blk["shared"] else None, blk["top"],
                                             blk["n_groups"], blk["keep_groups"])
                mode = self.moe_grouped
                if mode is None and torch.cuda.is_current_stream_capturing():
                    # a recorded decoding step keeps to this library's own kernels, whatever the batch size
                    mode = False if T * blk["top"] <= 256 else "own"
                ye, rows_e = nsq.moe_experts(h, idx, blk["w_gu"], blk["w_down"], grouped=mode) if blk["n_experts"] else (None, None)
                ys = None
                if blk["shared"]:
                    gu = nsq.linear(h, blk["ws_gu"])
                    ys = nsq.linear(nsq.silu_mul(gu, gu.shape[1] // 2), blk["ws_down"])
                nsq.moe_combine(x, ye, idx, wgt, h, blk["n_experts"], m, ys=ys, shared_gate=sg, y_row=rows_e)
            else:
                nsq.norm_conv(x, None, eps, None, y=y, y_mult=m)
            if self.layer_trace is not None:
                self.layer_trace.append(x.clone())
            if i + 1 < len(self.blocks):
                self._mixer_input(x, h, i + 1, batch)
        if rows is None or rows.numel() == 0:
            return torch.zeros(0, self.vocab_size, dtype=torch.float32, device=dev)
        hw = torch.empty(rows.numel(), W, dtype=dt, device=dev)
        nsq.rmsnorm(x, self.final_norm, hw, eps, rows=rows)
        return nsq.linear(hw, self.head).float()
