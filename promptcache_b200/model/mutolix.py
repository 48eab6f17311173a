"""Mutolix: a decoder-only model that interleaves matrix-memory recurrent layers (mLSTM) with attention layers.

Every sublayer is wrapped the same way (h = norm(x) goes in; the result is gated by sigmoid(W_rg h + b), RMS-normed,
scaled per channel and added to the 32-bit residual stream).  The mixers:

  mlstm       q, k, v and an output gate are projections of h; two capped gates per head drive a stabilised matrix-memory
              recurrence whose state lives in the slot pool (`pcs_mlstm_gates`, `pcs_mlstm_scan`);
  attention   grouped heads with distinct key and value widths, biased projections, RMS norm over the whole q and k
              projections, a position-dependent query temperature, no rotation, a logarithmic distance bias, one sink
              term in the softmax denominator, and values optionally mixed with those of the first such layer
              (`pcs_qk_prep`, `pcs_attn`).

The feed-forward is W_down xIELU(W_up h).  Projections (one per sublayer input with the gate's rows fused in, one per
sublayer output) are library matrix products for prompts and `pcs_linear_rows`, which streams the weights once, for the
one to eight rows of a decoding step; everything between them runs in the sequence-batch kernels.  Sizes, the
order of layers and every constant come from config.json; tensors are named l<i>.norm1, l<i>.mix.q, ... in the checkpoint.
"""
from __future__ import annotations

import json
import os
from typing import Dict, List, Optional

import torch

from .. import _native_seq as nsq
from .. import weights as wio
from ._seqbase import SlotPoolCausalLM
from ._state import KVSpec, MatrixMemorySpec


class MutolixConfig:
    """config.json of the design: {"architecture", "vocab", "width", "embedding": {"scale"}, "norm": {"eps"},
    "layers": [{"type": "mlstm" | "attention", "mixer": {...}, "mlp": {"kind": "dense", "ff"} | null}]}."""

    def __init__(self, d: dict):
        self.raw = d
        self.architecture = d.get("architecture", "Mutolix")
        self.vocab_size = int(d["vocab"])
        self.width = int(d["width"])
        self.embedding_scale = float(d.get("embedding", {}).get("scale", 1.0))
        self.eps = float(d.get("norm", {}).get("eps", 1e-6))
        self.layers = []
        for i, layer in enumerate(d["layers"]):
            kind = layer["type"]
            if kind not in ("mlstm", "attention"):
                raise ValueError(f"layer {i}: unknown mixer type {kind!r}")
            mlp = layer.get("mlp")
            if mlp is not None and mlp.get("kind", "dense") != "dense":
                raise ValueError(f"layer {i}: unknown feed-forward kind {mlp.get('kind')!r}")
            self.layers.append({"type": kind, "mixer": dict(layer["mixer"]), "mlp": dict(mlp) if mlp is not None else None})
        self.num_hidden_layers = len(self.layers)

    @classmethod
    def from_dir(cls, path: str) -> "MutolixConfig":
        with open(os.path.join(path, "config.json")) as fh:
            return cls(json.load(fh))


class MutolixForCausalLM(SlotPoolCausalLM):
    def __init__(self, config: MutolixConfig, tensors: Dict[str, torch.Tensor], device="cuda", dtype=torch.bfloat16,
                 max_tokens: Optional[int] = None):
        super().__init__()
        if dtype not in (torch.bfloat16, torch.float32):
            raise ValueError("Mutolix computes in bfloat16 or float32")
        self.config, self.compute_dtype = config, dtype
        self.vocab_size, self.width, self.eps = config.vocab_size, config.width, config.eps
        dev = torch.device(device)
        W = self.width

        def get(name, optional=False):
            t = tensors.get(name)
            if t is None:
                if optional:
                    return None
                raise KeyError(f"the checkpoint has no tensor {name!r}")
            return t.to(dev, dtype).contiguous()

        def f32(name):
            return tensors[name].to(dev, torch.float32).contiguous()

        def fuse(parts, biases):
            """Rows of several projections of the same input as one matrix; a missing bias is zero."""
            w = torch.cat(parts, 0).contiguous()
            if all(b is None for b in biases):
                return w, None
            b = torch.cat([bb if bb is not None else torch.zeros(p.shape[0], device=dev, dtype=dtype) for p, bb in zip(parts, biases)])
            return w, b.contiguous()

        self.embed = get("embed")
        self.final_norm, self.head = get("final.norm"), get("head")
        self.blocks: List[dict] = []
        self.first_vmix: Optional[int] = None
        for i, layer in enumerate(config.layers):
            p, m = f"l{i}.", layer["mixer"]
            blk = {"type": layer["type"], "norm1": get(p + "norm1"), "norm1b": get(p + "norm1b"), "ls1": get(p + "ls1", True)}
            rg, rgb = get(p + "rg1", True), get(p + "rg1.b", True)
            if layer["type"] == "mlstm":
                H, D, V = int(m["heads"]), int(m["dim"]), int(m["vdim"])
                parts = [get(p + "mix.q"), get(p + "mix.k"), get(p + "mix.v"), get(p + "mix.g")]
                offs = [0, H * D, 2 * H * D, 2 * H * D + H * V]
                blk.update(heads=H, dim=D, vdim=V, cap=float(m["gate_cap"]), offs=tuple(offs), rg_off=2 * H * D + 2 * H * V,
                           w_i=get(p + "mix.i"), w_f=get(p + "mix.f"), b_i=f32(p + "mix.i.b"), b_f=f32(p + "mix.f.b"),
                           mix_norm=get(p + "mix.norm"), w_o=get(p + "mix.o"), spec=MatrixMemorySpec(H, D, V))
                biases = [None] * 4
            else:
                H, D, V = int(m["heads"]), int(m["dim"]), int(m["vdim"])
                G = int(m.get("kv_heads", H))
                parts = [get(p + "mix.q"), get(p + "mix.k"), get(p + "mix.v")]
                biases = [get(p + "mix.q.b", True), get(p + "mix.k.b", True), get(p + "mix.v.b", True)]
                qt = m.get("q_temp") or {}
                mix_from = None
                if m.get("v_mix"):
                    if self.first_vmix is None:
                        self.first_vmix = i
                    else:
                        mix_from = self.first_vmix
                        f = config.layers[mix_from]["mixer"]
                        if (int(f.get("kv_heads", f["heads"])), int(f["vdim"])) != (G, V):
                            raise ValueError(f"layer {i}: value mixing needs the value shape of layer {mix_from}")
                r1, r2 = tensors.get(p + "mix.r1"), tensors.get(p + "mix.r2")
                blk.update(heads=H, kv_heads=G, dim=D, vdim=V, scale=float(m.get("scale", D ** -0.5)), offs=(0, H * D, (H + G) * D),
                           rg_off=(H + G) * D + G * V, q_norm=get(p + "mix.q.norm", True), k_norm=get(p + "mix.k.norm", True),
                           temp_coef=float(qt.get("coef", 0.0)), temp_every=int(qt.get("every", 0)) if qt else 0,
                           mix_from=mix_from, lam=get(p + "mix.vmix").reshape(1) if mix_from is not None else None,
                           r1=f32(p + "mix.r1") if r1 is not None else None, r2=f32(p + "mix.r2") if r2 is not None else None,
                           w_o=get(p + "mix.o"), spec=KVSpec(G, D, V))
            if rg is not None:
                parts.append(rg)
                biases.append(rgb)
            blk["gated1"] = rg is not None
            blk["w_in"], blk["b_in"] = fuse(parts, biases)
            if layer["mlp"] is not None:
                up = get(p + "mlp.up")
                rg2, rg2b = get(p + "rg2", True), get(p + "rg2.b", True)
                blk.update(ff=up.shape[0], norm2=get(p + "norm2"), norm2b=get(p + "norm2b"), ls2=get(p + "ls2", True),
                           act=get(p + "mlp.act"), w_down=get(p + "mlp.down"), gated2=rg2 is not None)
                blk["w_up"], blk["b_up"] = fuse([up] + ([rg2] if rg2 is not None else []), [None] + ([rg2b] if rg2 is not None else []))
            else:
                blk["ff"] = 0
            self.blocks.append(blk)
        # bfloat16 products accumulate in 32-bit all the way (no reduced-precision split-K sums); float32 stays true float32
        torch.backends.cuda.matmul.allow_bf16_reduced_precision_reduction = False
        torch.backends.cuda.matmul.allow_tf32 = False
        torch.backends.cudnn.allow_tf32 = False
        self.attn_impl = 0
        self.scan_impl = 0
        self._init_runtime(dev, max_tokens)

    def state_specs(self):
        return [b["spec"] for b in self.blocks]

    @classmethod
    def from_pretrained(cls, path: str, device="cuda", dtype=torch.bfloat16, max_tokens: Optional[int] = None, **_):
        """`path`: a folder with config.json and model.safetensors."""
        cfg = MutolixConfig.from_dir(path)
        tensors = wio.load_file(os.path.join(path, "model.safetensors"), device=device)
        return cls(cfg, tensors, device=device, dtype=dtype, max_tokens=max_tokens)

    # ---- the layers over one batch ------------------------------------------------------------------------------
    def _layers(self, ids: torch.Tensor, batch, rows: Optional[torch.Tensor]) -> torch.Tensor:
        T, W, dt, dev, eps = ids.shape[0], self.width, self.compute_dtype, self._device, self.eps
        x = torch.empty(T, W, dtype=torch.float32, device=dev)     # the residual stream, 32-bit, updated in place
        h = torch.empty(T, W, dtype=dt, device=dev)                # the normed input of the next sublayer
        nsq.embed(self.embed, ids, x, self.config.embedding_scale)
        nsq.rmsnorm(x, self.blocks[0]["norm1"], h, eps)
        for i, blk in enumerate(self.blocks):
            st = self.pool.layers[i]
            nxt = self.blocks[i + 1]["norm1"] if i + 1 < len(self.blocks) else None
            proj = nsq.linear(h, blk["w_in"], blk["b_in"])
            H, V = blk["heads"], blk["vdim"]
            mixed = torch.empty(T, H * V, dtype=dt, device=dev)
            if blk["type"] == "mlstm":
                ig = torch.empty(T, H, dtype=torch.float32, device=dev)
                fg = torch.empty(T, H, dtype=torch.float32, device=dev)
                nsq.mlstm_gates(h, blk["w_i"], blk["w_f"], blk["b_i"], blk["b_f"], ig, fg, blk["cap"])
                nsq.mlstm_scan(proj, blk["offs"], ig, fg, blk["mix_norm"], mixed, st["s"], st["n"], st["m"], eps, batch,
                               impl=self.scan_impl)
            else:
                q = torch.empty(T, H * blk["dim"], dtype=dt, device=dev)
                vf = self.pool.layers[blk["mix_from"]]["v"] if blk["mix_from"] is not None else None
                nsq.qk_prep(proj, blk["offs"], blk["q_norm"], blk["k_norm"], eps, H, blk["kv_heads"], blk["dim"], V, blk["temp_coef"],
                            blk["temp_every"], q, st["k"], st["v"], vf, blk["lam"], batch)
                # few tokens (decoding): the keys are split over more blocks; the bound is the pool's capacity, so that a
                # replayed graph stays valid while the sequences grow
                ws = nsq.attn_workspace(T, H, V, dev) if T <= 16 else None
                nsq.attention(q, st["k"], st["v"], mixed, H, blk["scale"], blk["r1"], blk["r2"], True, batch, impl=self.attn_impl,
                              max_keys=self.pool.cap, workspace=ws)
            y = nsq.linear(mixed, blk["w_o"])
            gate = proj[:, blk["rg_off"]:] if blk["gated1"] else None
            has_ff = blk["ff"] > 0
            nsq.gate_norm_add(x, y, gate, blk["norm1b"], blk["ls1"], eps, blk["norm2"] if has_ff else nxt, h if (has_ff or nxt is not None) else None)
            if has_ff:
                ff = blk["ff"]
                u = nsq.linear(h, blk["w_up"], blk["b_up"])
                a = torch.empty(T, ff, dtype=dt, device=dev)
                nsq.xielu(u[:, :ff], a, blk["act"])
                d = nsq.linear(a, blk["w_down"])
                nsq.gate_norm_add(x, d, u[:, ff:] if blk["gated2"] else None, blk["norm2b"], blk["ls2"], eps, nxt, h if nxt is not None else None)
            if self.layer_trace is not None:
                self.layer_trace.append(x.clone())
        if rows is None or rows.numel() == 0:
            return torch.zeros(0, self.vocab_size, dtype=torch.float32, device=dev)
        hw = torch.empty(rows.numel(), W, dtype=dt, device=dev)
        nsq.rmsnorm(x, self.final_norm, hw, eps, rows=rows)
        return nsq.linear(hw, self.head).float()
