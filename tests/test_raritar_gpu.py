"""The Raritar design on the GPU against the float64 oracle (tests/raritar_oracle.py): each mechanism alone through the
kernels' bindings, then whole models through the step function, the batch engine, the generation engine and bin/trace_run."""
import json
import math
import os
import subprocess
import sys

import pytest
import torch

from tests import raritar_oracle as O

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
F32, BF16, F64 = torch.float32, torch.bfloat16, torch.float64
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def nsq():
    from promptcache_b200 import _native_seq
    _native_seq.load()
    return _native_seq


def dev(t, dtype=F32):
    return t.to(DEV, dtype).contiguous()


def close(got, want, tol, what=""):
    got, want = got.detach().cpu().to(F64), want.to(F64)
    err = float((got - want).abs().max() / (want.abs().max() + 1e-30))
    assert err <= tol, f"{what}: relative error {err:.3e} > {tol:.1e}"
    return err


def close_rms(got, want, tol, what=""):
    got, want = got.detach().cpu().to(F64), want.detach().cpu().to(F64)
    err = float((got - want).pow(2).mean().sqrt() / want.pow(2).mean().sqrt())
    assert err <= tol, f"{what}: relative rms error {err:.3e} > {tol:.1e}"
    return err


def close_rows(got, want, tol, what="", share=0.85, worst=0.6):
    """bfloat16 runs of whole models: a rounding can flip a router's choice between two near-equal experts, which moves that
    token's logits by far more than rounding does.  So rows are judged one by one: most of them within `tol` (relative root
    mean square), none beyond `worst`."""
    got, want = got.detach().cpu().to(F64), want.detach().cpu().to(F64)
    err = (got - want).pow(2).mean(-1).sqrt() / want.pow(2).mean(-1).sqrt()
    ok = float((err <= tol).double().mean())
    assert ok >= share and float(err.max()) <= worst, f"{what}: {ok:.2f} of the rows within {tol:.1e}, worst {float(err.max()):.3e}"


def write_checkpoint(folder, cfg, W):
    from promptcache_b200 import weights as wio
    os.makedirs(folder, exist_ok=True)
    with open(os.path.join(folder, "config.json"), "w") as fh:
        json.dump(cfg, fh)
    wio.save_file({k: v.to(BF16) for k, v in W.items()}, os.path.join(folder, "model.safetensors"))


def load(tmp_path, cfg, W, dtype=F32, name="m"):
    from promptcache_b200.model import load_model
    folder = str(tmp_path / name)
    write_checkpoint(folder, cfg, W)
    return load_model(folder, device=DEV, dtype=dtype)


def tokens(n, vocab, seed):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (n,), generator=g).tolist()


def batch_of(nsq, slots, pos0, lens, parity=None):
    return nsq.Batch(slots, pos0, lens, torch.device(DEV), parity)


# ---- mechanisms alone ---------------------------------------------------------------------------------------------
def test_pair_embedding(nsq):
    torch.manual_seed(0)
    vocab, width, buckets, mp, mc = 37, 24, 11, 29, 5
    table, pair = torch.randn(vocab, width, dtype=F64), torch.randn(buckets + 1, width, dtype=F64)
    toks = tokens(9, vocab, 1)
    want = table[toks] + pair[O.bigram_rows(toks, buckets, mp, mc)]
    ids = torch.tensor(toks, device=DEV)
    prev = torch.tensor([-1] + toks[:-1], device=DEV)
    out = torch.empty(9, width, device=DEV)
    nsq.embed_bigram(dev(table), dev(pair), ids, prev, out, buckets, mp, mc)
    close(out, want, 1e-6, "pair embedding")
    # multipliers larger than the table and a continued sequence (the predecessor comes from the caller)
    big_p, big_c = 10 ** 12 + 3, 10 ** 9 + 7
    rows = [(a * big_p + b * big_c) % buckets for a, b in zip(toks[:-1], toks[1:])]
    nsq.embed_bigram(dev(table), dev(pair), ids[1:].contiguous(), ids[:-1].contiguous(), out[1:], buckets, big_p, big_c)
    close(out[1:], table[toks[1:]] + pair[rows], 1e-6, "pair embedding, large multipliers")


@pytest.mark.parametrize("taps,width", [(4, 40), (2, 33), (1, 16), (8, 24), (4, 1536), (3, 2052)])
def test_norm_and_time_convolution_in_portions(nsq, taps, width):
    """Whole sequence at once against portions of every small size, through a dirty reused slot, two sequences interleaved."""
    torch.manual_seed(taps)
    T, eps = 19, 1e-5
    g = torch.tensor([1.3], dtype=F64)
    w = torch.randn(width, taps, dtype=F64) * 0.5
    xs = [torch.randn(T, width, dtype=F64) * 2, torch.randn(T, width, dtype=F64)]
    want = []
    for x in xs:
        u = O.rms(x, eps) * g
        want.append(u + O.time_conv(u, w))
    tail = torch.full((3, 2, max(taps - 1, 1), width), 7.0, device=DEV)   # dirty: nothing may be read before a sequence's start
    for cuts in ([T], [1] * T, [2, 1, 3, 2, 5, 6], [5, 1, 1, 1, 11]):
        got = [[], []]
        pos, steps = [0, 0], [0, 0]
        for i, n in enumerate(cuts):
            # the two sequences run in one batch, the second one step behind at first (different parities)
            entries = [0, 1] if i > 0 else [0]
            lens = [n if b == 0 else cuts[i - 1] for b in entries]
            x = torch.cat([xs[b][pos[b]:pos[b] + l] for b, l in zip(entries, lens)])
            h = torch.empty(x.shape[0], width, device=DEV)
            b_ = batch_of(nsq, [2 if b == 0 else 0 for b in entries], [pos[b] for b in entries], lens, [steps[b] & 1 for b in entries])
            nsq.norm_conv(dev(x), dev(g), eps, h, conv_w=dev(w.t()), tail=tail, batch=b_)
            o = 0
            for b, l in zip(entries, lens):
                got[b].append(h[o:o + l].cpu())
                o += l
                pos[b] += l
                steps[b] += 1
        close(torch.cat(got[0]), want[0], 3e-6, f"norm + convolution, cuts {cuts}")
        if got[1]:
            close(torch.cat(got[1]), want[1][:sum(cuts[:-1])], 3e-6, f"norm + convolution of the second sequence, cuts {cuts}")


def test_norm_with_residual_sum(nsq):
    torch.manual_seed(3)
    T, width, eps = 6, 72, 1e-5
    x, y = torch.randn(T, width, dtype=F64), torch.randn(T, width, dtype=F64)
    gvec = torch.randn(width, dtype=F64)
    xd, h = dev(x), torch.empty(T, width, device=DEV)
    nsq.norm_conv(xd, dev(gvec), eps, h, y=dev(y), y_mult=0.65)
    close(xd, x + 0.65 * y, 1e-6, "residual sum")
    close(h, O.rms(x + 0.65 * y, eps) * gvec, 3e-6, "norm with one weight per channel")
    xd2 = dev(x)
    nsq.norm_conv(xd2, None, eps, None, y=dev(y), y_mult=-1.5)
    close(xd2, x - 1.5 * y, 1e-6, "residual sum alone")


@pytest.mark.parametrize("rot,dim,scaling", [(8, 16, True), (16, 16, False), (0, 8, False), (6, 10, True)])
def test_rotation_value_norm_and_append(nsq, rot, dim, scaling):
    torch.manual_seed(rot + dim)
    H, G, V, T, eps, cap = 4, 2, 12, 7, 1e-5, 128
    sc = {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 64} if scaling else None
    freqs = O.rotary_frequencies(rot, 10000.0, sc)
    from promptcache_b200.model.raritar import scaled_frequencies
    assert scaled_frequencies(rot, 10000.0, sc) == pytest.approx(freqs, rel=1e-14)
    pos = [0, 1, 2, 100000, 100001, 5, 6]     # two entries; one far along, where a 32-bit angle would have lost its low bits
    qkv = torch.randn(T, (H + G) * dim + G * V, dtype=F64)
    q = O.rotate(qkv[:, :H * dim].view(T, H, dim), pos, freqs)
    k = O.rotate(qkv[:, H * dim:(H + G) * dim].view(T, G, dim), pos, freqs)
    v = O.rms(qkv[:, (H + G) * dim:].view(T, G, V), eps)
    b = batch_of(nsq, [1, 0], [0, 100000], [3, 2])
    kp, vp = torch.zeros(2, G, 100096, dim, device=DEV), torch.zeros(2, G, 100096, V, device=DEV)
    qo = torch.empty(5, H * dim, device=DEV)
    fd = torch.tensor(freqs, dtype=F64, device=DEV) if rot else None
    nsq.rope_kv_prep(dev(qkv[:5]), (0, H * dim, (H + G) * dim), H, G, dim, V, fd, rot, True, True, eps, qo, kp, vp, b)
    close(qo.view(5, H, dim), q[:5], 2e-6, "rotated queries")
    close(kp[1, :, 0:3].transpose(0, 1), k[:3], 2e-6, "rotated keys in the pool")
    close(kp[0, :, 100000:100002].transpose(0, 1), k[3:5], 2e-6, "rotated keys far along")
    close(vp[1, :, 0:3].transpose(0, 1), v[:3], 2e-6, "unit-RMS values in the pool")
    # a layer without rows of its own only rotates its queries
    kp2 = kp.clone()
    nsq.rope_kv_prep(dev(qkv[:5, :H * dim]), (0, None, None), H, G, dim, V, fd, rot, True, True, eps, qo, None, None, b)
    assert torch.equal(kp, kp2)
    close(qo.view(5, H, dim), q[:5], 2e-6, "queries of a layer that reads another layer's rows")


def run_attention(nsq, q, k, v, window, keep_first, softcap, scale, dtype, impl=0, pos0=0, decode=False):
    """q [T, H, D] are the LAST T tokens of a sequence whose keys k [N, G, D] / values are all cached."""
    T, H, D = q.shape
    N, G, V = k.shape[0], k.shape[1], v.shape[2]
    cap = (N + 127) // 128 * 128
    kp, vp = torch.zeros(2, G, cap, D, device=DEV, dtype=dtype), torch.zeros(2, G, cap, V, device=DEV, dtype=dtype)
    kp[1, :, :N] = dev(k, dtype).transpose(0, 1)
    vp[1, :, :N] = dev(v, dtype).transpose(0, 1)
    out = torch.empty(T, H * V, device=DEV, dtype=dtype)
    b = batch_of(nsq, [1], [N - T], [T])
    ws = nsq.attn_workspace(T, H, V, DEV) if decode else None
    seen = min(cap, window + keep_first) if window > 0 else cap
    nsq.attention(dev(q.reshape(T, H * D), dtype), kp, vp, out, H, scale, None, None, False, b, impl=impl, max_keys=seen, workspace=ws,
                  softcap=softcap, window=window, keep_first=keep_first)
    return out.view(T, H, V)


@pytest.mark.parametrize("window,keep_first,softcap", [(48, 5, 45.0), (64, 0, 0.0), (1, 2, 20.0), (0, 0, 30.0), (100, 70, 10.0), (700, 5, 0.0)])
def test_windowed_attention_kernels(nsq, window, keep_first, softcap):
    """The plain kernel (32-bit), the tensor-core kernel (prompts, bfloat16) and the split-key kernel (decoding) against the
    oracle, over tile borders of 64 and 128 keys."""
    torch.manual_seed(window + keep_first)
    H, G, D, V, N = 4, 2, 16, 24, 333
    q, k, v = torch.randn(N, H, D, dtype=F64), torch.randn(N, G, D, dtype=F64), torch.randn(N, G, V, dtype=F64)
    scale = 1.7 / math.sqrt(D)
    w = window if window > 0 else 1 << 30
    want = O.attention_core(q, k, v, scale, softcap, w, keep_first)
    got = run_attention(nsq, q, k, v, window, keep_first, softcap, scale, F32, impl=1)
    close(got, want, 1e-5, "plain kernel, whole prompt")
    qb, kb, vb = (t.to(BF16).to(F64) for t in (q, k, v))
    want_b = O.attention_core(qb, kb, vb, scale, softcap, w, keep_first)
    got = run_attention(nsq, qb, kb, vb, window, keep_first, softcap, scale, BF16)
    close(got, want_b, 1.5e-2, "tensor-core kernel, whole prompt")
    close_rms(got, want_b, 4e-3, "tensor-core kernel, whole prompt")
    for T in (70, 17):   # a portion on top of cached keys
        got = run_attention(nsq, qb[N - T:], kb, vb, window, keep_first, softcap, scale, BF16)
        close_rms(got, want_b[N - T:], 4e-3, f"tensor-core kernel, last {T} tokens")
        got = run_attention(nsq, q[N - T:], k, v, window, keep_first, softcap, scale, F32)
        close(got, want[N - T:], 1e-5, f"plain kernel, last {T} tokens")
    for n in (N, 129, 128, 65, 41, 5, 1):   # decoding: one query over n cached keys
        got = run_attention(nsq, q[n - 1:n], k[:n], v[:n], window, keep_first, softcap, scale, F32, decode=True)
        close(got, want[n - 1:n], 1e-5, f"split-key kernel, {n} keys")
        got = run_attention(nsq, qb[n - 1:n], kb[:n], vb[:n], window, keep_first, softcap, scale, BF16, decode=True)
        close(got, want_b[n - 1:n], 1.5e-2, f"split-key kernel in bfloat16, {n} keys")


@pytest.mark.parametrize("dtype", [F32, BF16])
def test_one_key_decides_at_every_edge(nsq, dtype):
    """One key is made to dominate (its query and key are scaled up) and carries a marked value: the result shows whether the
    key was seen.  Just inside / outside the window, the last kept first key / the next one, keys far back, at tile borders,
    in a prompt and in decoding."""
    H, G, D, V, N = 2, 1, 16, 8, 420
    window, keep_first = 50, 3
    g = torch.Generator().manual_seed(5)
    scale = 1.0
    for i, j, seen in [(419, 370, True), (419, 369, False), (419, 2, True), (419, 3, False), (419, 0, True), (300, 251, True),
                       (300, 250, False), (128, 79, True), (128, 78, False), (64, 15, True), (64, 14, False), (63, 63, True),
                       (191, 128, False), (255, 206, True), (49, 0, True), (52, 3, True), (53, 3, False)]:
        q = torch.randn(N, H, D, generator=g, dtype=F64) * 0.1
        k = torch.randn(N, G, D, generator=g, dtype=F64) * 0.1
        v = torch.randn(N, G, V, generator=g, dtype=F64) * 0.1
        d = torch.zeros(D, dtype=F64)
        d[5] = 6.0
        q[i, :] = d
        k[j, 0] = d          # score 36 against scores near 0
        v[j, 0] = 9.0
        q, k, v = (t.to(BF16).to(F64) for t in (q, k, v))
        want = O.attention_core(q[:i + 1], k[:i + 1], v[:i + 1], scale, 0.0, window, keep_first)[i]
        assert (want.mean() > 8.0) == seen
        got = run_attention(nsq, q[:i + 1], k[:i + 1], v[:i + 1], window, keep_first, 0.0, scale, dtype)[i]
        close(got, want, 1e-2 if dtype == BF16 else 1e-5, f"prompt, query {i} key {j}")
        got = run_attention(nsq, q[i:i + 1], k[:i + 1], v[:i + 1], window, keep_first, 0.0, scale, dtype, decode=True)[0]
        close(got, want, 1e-2 if dtype == BF16 else 1e-5, f"decoding, query {i} key {j}")
        if i > 40:
            got = run_attention(nsq, q[i - 30:i + 1], k[:i + 1], v[:i + 1], window, keep_first, 0.0, scale, dtype)[30]
            close(got, want, 1e-2 if dtype == BF16 else 1e-5, f"portion, query {i} key {j}")


@pytest.mark.parametrize("E,I,top,groups,keep", [(6, 2, 3, 4, 2), (8, 0, 2, 1, 1), (5, 1, 2, 3, 1), (4, 4, 4, 2, 1), (64, 0, 8, 8, 3), (3, 0, 3, 1, 1)])
def test_router(nsq, E, I, top, groups, keep):
    torch.manual_seed(E * 7 + top)
    T, W = 100, 48                                        # many tokens: one warp per token; few (below): one block per token
    h = torch.randn(T, W, dtype=F64)
    wr = torch.randn(E + I, W, dtype=F64) * 0.5
    corr = torch.randn(E + I, dtype=F64) * 0.2 - 0.3      # negative choice scores: a masked output must not win as "0"
    wsg = torch.randn(W, dtype=F64) * 0.3
    idx, wgt, sg = nsq.moe_route(dev(h), dev(wr), dev(corr), dev(wsg), top, groups, keep)
    close(sg, torch.sigmoid(h @ wsg), 1e-5, "shared gate")
    z = h @ wr.T
    for t in range(T):
        chosen, ws = O.route(z[t], corr, top, groups, keep)
        assert idx[t].tolist() == chosen, f"token {t}: chose {idx[t].tolist()}, oracle {chosen}"
        close(wgt[t], torch.stack(ws), 1e-5, "router weights")
    idx5, wgt5, sg5 = nsq.moe_route(dev(h[:5]), dev(wr), dev(corr), dev(wsg), top, groups, keep)
    assert torch.equal(idx5, idx[:5]) and torch.equal(wgt5, wgt[:5]) and torch.equal(sg5, sg[:5])
    idx2, wgt2, none = nsq.moe_route(dev(h), dev(wr), None, None, top, groups, keep)
    assert none is None
    chosen, _ = O.route(z[0], torch.zeros(E + I, dtype=F64), top, groups, keep)
    assert idx2[0].tolist() == chosen


@pytest.mark.parametrize("T,ff,W", [(3, 24, 40), (150, 40, 72), (70, 20, 36)])
def test_experts_rows_grouped_and_combine(nsq, T, ff, W):
    torch.manual_seed(T)
    E, I, top = 5, 2, 3
    Wt = {}
    for e in range(E):
        Wt[f"e{e}.gate"], Wt[f"e{e}.up"], Wt[f"e{e}.down"] = (torch.randn(ff, W, dtype=F64) * 0.3, torch.randn(ff, W, dtype=F64) * 0.3,
                                                            torch.randn(W, ff, dtype=F64) * 0.3)
    Wt = {k_: v_.to(BF16).to(F64) for k_, v_ in Wt.items()}
    h = (torch.randn(T, W, dtype=F64)).to(BF16).to(F64)
    g = torch.Generator().manual_seed(1)
    idx = torch.stack([torch.randperm(E + I, generator=g)[:top] for _ in range(T)]).to(torch.int32)
    if T > 100:
        idx[:, 0] = 1                                     # one expert gets more than a tile of rows; expert 4 may get none
        idx[idx == 4] = 6
    w_gu = torch.stack([torch.cat([Wt[f"e{e}.gate"], Wt[f"e{e}.up"]]) for e in range(E)])
    w_dn = torch.stack([Wt[f"e{e}.down"] for e in range(E)])
    want = torch.zeros(T * top, W, dtype=F64)
    real = torch.zeros(T * top, dtype=torch.bool)
    for t in range(T):
        for k_ in range(top):
            e = int(idx[t, k_])
            if e < E:
                want[t * top + k_] = O.gated_ff(Wt, f"e{e}.", h[t:t + 1])[0]
                real[t * top + k_] = True
    rd = real.to(DEV)
    y32, none = nsq.moe_experts(dev(h), idx.to(DEV), dev(w_gu), dev(w_dn), grouped=False)
    assert none is None
    close(y32[rd], want[real], 1e-5, "row kernels, 32-bit")
    yb, _ = nsq.moe_experts(dev(h, BF16), idx.to(DEV), dev(w_gu, BF16), dev(w_dn, BF16), grouped=False)
    close_rms(yb[rd], want[real], 4e-3, "row kernels, bfloat16")
    if ff % 8 or W % 8:                                   # sizes the 16-byte copies cannot take stay with the row kernels
        with pytest.raises(nsq.NativeError):
            nsq.moe_experts(dev(h, BF16), idx.to(DEV), dev(w_gu, BF16), dev(w_dn, BF16), grouped="library")
    else:
        yg, none = nsq.moe_experts(dev(h, BF16), idx.to(DEV), dev(w_gu, BF16), dev(w_dn, BF16), grouped="own")
        assert none is None
        close_rms(yg[rd], want[real], 4e-3, "own grouped products")
        close_rms(yg[rd], yb[rd], 2e-3, "own grouped products against the row kernels")
        yl, row_of = nsq.moe_experts(dev(h, BF16), idx.to(DEV), dev(w_gu, BF16), dev(w_dn, BF16), grouped="library")
        assert bool((row_of[rd] >= 0).all()) and bool((row_of[~rd] == -1).all())
        assert sorted(row_of[rd].tolist()) == list(range(int(real.sum())))      # the sort is a permutation of the real pairs
        e_sorted = idx.flatten()[real][torch.argsort(row_of[rd].cpu())]
        assert bool((e_sorted[1:] >= e_sorted[:-1]).all())                      # ... by expert
        close_rms(yl[row_of[rd].long()], want[real], 8e-3, "library grouped products on sorted rows")
        xa, xb = torch.zeros(T, W, device=DEV), torch.zeros(T, W, device=DEV)
        ones = torch.ones(T, top, device=DEV)
        nsq.moe_combine(xa, yl, idx.to(DEV), ones, dev(h, BF16), E, 1.0, y_row=row_of)
        nsq.moe_combine(xb, yg, idx.to(DEV), ones, dev(h, BF16), E, 1.0)
        close_rms(xa, xb, 8e-3, "weighted sum through the row map")
    # the weighted sum with pass-through outputs and the gated shared expert
    x = torch.randn(T, W, dtype=F64)
    wgt, sg, ys = torch.rand(T, top, dtype=F64), torch.rand(T, dtype=F64), torch.randn(T, W, dtype=F64)
    exp = x.clone()
    for t in range(T):
        a = sg[t] * ys[t]
        for k_ in range(top):
            a = a + wgt[t, k_] * (want[t * top + k_] if real[t * top + k_] else h[t])
        exp[t] += 0.65 * a
    xd = dev(x)
    y_in = dev(want)
    y_in[~real.to(DEV)] = float("nan")                    # rows of pass-through choices are never read
    nsq.moe_combine(xd, y_in, idx.to(DEV), dev(wgt), dev(h), E, 0.65, ys=dev(ys), shared_gate=dev(sg))
    close(xd, exp, 2e-6, "weighted sum into the residual stream")
    gu = torch.randn(T, 2 * ff, dtype=F64)
    close(nsq.silu_mul(dev(gu), ff), O.silu(gu[:, :ff]) * gu[:, ff:], 2e-6, "silu(gate) * up")


# ---- whole models ---------------------------------------------------------------------------------------------------
def layer_sets():
    A = O.attn_layer
    return {
        "mixed": [A(), A(heads=2, kv_heads=2, dim=8, vdim=16, window=7, keep_first=0, rot_dims=8, scaling=False, softcap=0.0, identity=0,
                    experts=4, top=2, groups=(1, 1), shared_ff=0),
                  A(kv_from=0, window=5, keep_first=1), A(kv_from=0, mlp=False), A(heads=1, kv_heads=1, dim=24, vdim=8, rot_dims=24, window=1000,
                                                                                   experts=2, identity=3, top=2, groups=(5, 3), ff=8, shared_ff=40)],
        # sizes that are not multiples of the 16-byte pieces: every kernel's plain path
        "odd": [A(heads=3, kv_heads=1, dim=12, vdim=20, rot_dims=6, window=6, keep_first=2, experts=3, identity=1, top=2, groups=(2, 1), ff=20,
                  shared_ff=12),
                A(heads=3, kv_heads=1, dim=12, vdim=20, rot_dims=6, window=11, keep_first=0, kv_from=0, experts=5, identity=0, top=3,
                  groups=(1, 1), ff=12, shared_ff=0)],
        "shared_first": [A(window=9, keep_first=2, top=1), A(kv_from=0, window=9, keep_first=2), A(kv_from=0, window=30, keep_first=0)],
    }


@pytest.mark.parametrize("name,taps,buckets,width", [("mixed", 4, 53, 40), ("mixed", 2, 0, 24), ("shared_first", 0, 7, 64), ("shared_first", 3, 1, 40), ("odd", 5, 10, 36),
                                                      ("odd", 9, 3, 30)])
def test_model_whole_prompt_against_oracle(tmp_path, name, taps, buckets, width):
    cfg = O.make_config(layer_sets()[name], width=width, taps=taps, buckets=buckets)
    W = O.random_model(cfg, seed=width)
    toks = tokens(45, cfg["vocab"], 2)
    trace = []
    want = O.forward(cfg, W, toks, trace)
    m = load(tmp_path, cfg, W, F32)
    m.layer_trace = []
    seq = m.new_sequence()
    got = m.step([(seq, toks)], [list(range(len(toks)))])
    for i, (a, b) in enumerate(zip(m.layer_trace, trace)):
        close(a, b, 3e-5, f"residual stream after layer {i}")
    close(got, want, 5e-5, "logits, float32")
    mb = load(tmp_path, cfg, W, BF16, "b")
    gb = mb.step([(mb.new_sequence(), toks)], [list(range(len(toks)))])
    close_rows(gb, want, 4e-2, "logits, bfloat16", share=0.7)


@pytest.mark.parametrize("dtype,tol", [(F32, 5e-5), (BF16, 4e-2)])
def test_portions_decoding_batches_and_slot_reuse(tmp_path, dtype, tol):
    """One set of sequences run whole, in portions of several sizes down to two tokens, token by token (through the
    replayed graph), in unequal batches whose shorter members leave early, and through slots that were used before."""
    cfg = O.make_config(layer_sets()["mixed"])
    W = O.random_model(cfg, seed=11)
    V = cfg["vocab"]
    seqs = [tokens(n, V, 20 + n) for n in (61, 9, 30, 1)]
    want = [O.forward(cfg, W, s) for s in seqs]
    m = load(tmp_path, cfg, W, dtype)
    cmp = close if dtype == F32 else close_rows

    def run(toks, cuts):
        seq, out, p = m.new_sequence(), [], 0
        for n in cuts:
            out.append(m.step([(seq, toks[p:p + n])], [list(range(n))]))
            p += n
        seq.free()
        return torch.cat(out)

    for cuts in ([61], [2] * 30 + [1], [1] * 61, [17, 2, 3, 1, 1, 30, 7], [40] + [1] * 21):
        cmp(run(seqs[0], cuts), want[0], tol, f"portions {cuts[:6]}...")
    # unequal batch: prompts together, then decoded together; the short ones leave earlier
    from promptcache_b200.batch_engine import BatchEngine
    eng = BatchEngine(m)
    pre = [40, 4, 22, 1]
    got = [[] for _ in seqs]
    lg = eng.step([(f"r{i}", s[:n], list(range(n))) for i, (s, n) in enumerate(zip(seqs, pre))])
    o = 0
    for i, n in enumerate(pre):
        got[i].append(lg[o:o + n])
        o += n
    at = list(pre)
    while any(a < len(s) for a, s in zip(at, seqs)):
        live = [i for i, s in enumerate(seqs) if at[i] < len(s)]
        done = [f"r{i}" for i in live if at[i] + 1 == len(seqs[i])]
        lg = eng.step([(f"r{i}", [seqs[i][at[i]]], [0]) for i in live], done)
        for k_, i in enumerate(live):
            got[i].append(lg[k_:k_ + 1])
            at[i] += 1
    eng.end("r3")
    for i in range(len(seqs)):
        cmp(torch.cat(got[i]), want[i], tol, f"request {i} in a batch")
    # the freed slots are handed out again, to other sequences and in another order
    lg = eng.step([("x", seqs[2], None), ("y", seqs[0], None), ("z", seqs[1], None)], ["x", "y", "z"])
    (close if dtype == F32 else close_rms)(lg, torch.stack([want[2][-1], want[0][-1], want[1][-1]]), tol if dtype == F32 else 0.1, "reused slots")


def test_long_decoding_past_window_and_pool_growth(tmp_path):
    """300 tokens decoded one by one after a short prompt: the window passes over decoded tokens, the pool grows twice while
    the sequence lives (captured graphs are rebuilt), and a second sequence joins and leaves."""
    cfg = O.make_config([O.attn_layer(window=40, keep_first=4), O.attn_layer(kv_from=0, window=64, keep_first=0), O.attn_layer(window=129, keep_first=1)])
    W = O.random_model(cfg, seed=3)
    toks = tokens(330, cfg["vocab"], 8)
    want = O.forward(cfg, W, toks)
    m = load(tmp_path, cfg, W, F32)
    seq = m.new_sequence()
    out = [m.step([(seq, toks[:30])], [list(range(30))])]
    other = None
    for p in range(30, 330):
        if p == 100:
            other = m.new_sequence()
            m.step([(other, toks[:50])])
        if other is not None and 100 <= p < 140:
            lg = m.step([(seq, [toks[p]]), (other, [toks[p - 50]])])
            close(lg[1], want[p - 50], 5e-5, f"second sequence at {p - 50}")
            out.append(lg[:1])
        else:
            if other is not None and p == 140:
                other.free()
            out.append(m.step([(seq, [toks[p]])]))
    close(torch.cat(out), want, 5e-5, "long decoding")


def test_medium_model_long_prompt(tmp_path):
    """Sizes at which the other code paths run: 64-wide heads on the tensor-core kernel over twenty key tiles, windows that skip
    tiles, a layer without a window whose decoding splits the keys, hundreds of pairs per expert through the grouped products."""
    A = O.attn_layer
    kw = dict(heads=8, kv_heads=2, dim=64, vdim=64, rot_dims=32, experts=8, identity=1, top=2, groups=(3, 2), ff=128, shared_ff=256)
    cfg = O.make_config([A(window=200, keep_first=5, **kw), A(window=5000, keep_first=0, **kw), A(window=130, keep_first=70, kv_from=1, **kw)],
                        width=256, vocab=300, buckets=211)
    W = O.random_model(cfg, seed=21)
    toks = tokens(1320, 300, 4)
    rows = list(range(0, 1300, 97)) + [1297, 1298, 1299]
    want = O.forward(cfg, W, toks)
    for dtype in (F32, BF16):
        m = load(tmp_path, cfg, W, dtype, str(dtype)[-4:])
        seq = m.new_sequence()
        got = [m.step([(seq, toks[:1300])], [rows])]
        for p_ in range(1300, 1320):
            got.append(m.step([(seq, [toks[p_]])]))
        got = torch.cat(got)
        ref = want[rows + list(range(1300, 1320))]
        if dtype == F32:
            close(got, ref, 1e-4, "medium model, float32")
        else:
            close_rows(got, ref, 5e-2, "medium model, bfloat16", share=0.7)
        seq.free()


def test_greedy_generation_through_the_engines(tmp_path):
    from promptcache_b200.batch_engine import BatchEngine
    from promptcache_b200.generation_engine import GenerationEngine, GenerationParameters
    from promptcache_b200.model import Raritar
    cfg = O.make_config(layer_sets()["shared_first"], width=48)
    W = O.random_model(cfg, seed=5)
    prompts = [tokens(n, cfg["vocab"], 40 + n) for n in (12, 3, 25)]
    n_new = 10

    def greedy(p):
        s = list(p)
        for _ in range(n_new):
            s.append(int(O.forward(cfg, W, s)[-1].argmax()))
        return s[len(p):]

    want = [greedy(p) for p in prompts]
    folder = str(tmp_path / "g")
    write_checkpoint(folder, cfg, W)
    lm = Raritar(folder, device=DEV, dtype=F32)
    params = GenerationParameters(temperature=0.0, max_new_tokens=n_new, stop_token_ids=[], stop_str=[])
    assert BatchEngine(lm.hf_model, max_tokens=4096).generate(prompts, params) == want
    for p, w in zip(prompts, want):
        outs = list(GenerationEngine(lm).generate(p, list(range(len(p))), params, None, stream_interval=2))
        assert outs[-1].new_text == lm.decode(w)
    assert not lm.hf_model.pool.rows                         # the engines gave their slots back
    stop = want[2][3]
    stopped = BatchEngine(lm.hf_model, max_tokens=64).generate(prompts, GenerationParameters(temperature=0.0, max_new_tokens=n_new, stop_token_ids=[stop]))
    assert stopped[2] == want[2][:want[2].index(stop) + 1]


def test_trace_replay_end_to_end(tmp_path):
    cfg = O.make_config(layer_sets()["mixed"])
    W = O.random_model(cfg, seed=9)
    folder = str(tmp_path / "t")
    write_checkpoint(folder, cfg, W)
    a, b = tokens(20, cfg["vocab"], 1), tokens(7, cfg["vocab"], 2)
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": a[:15], "want": [0, 14]}, {"id": "b", "tokens": b[:6], "want": []}], "end": []},
             {"step": 1, "entries": [{"id": "a", "tokens": a[15:16], "want": [0]}, {"id": "b", "tokens": b[6:], "want": [0]}], "end": ["b"]}] + \
            [{"step": 2 + i, "entries": [{"id": "a", "tokens": [a[16 + i]], "want": [0]}], "end": ["a"] if i == 3 else []} for i in range(4)]
    out = str(tmp_path / "out")
    r = subprocess.run([os.path.join(ROOT, "bin", "trace_run"), "--model", folder, "--dtype", "float32", "--out", out, "--max-tokens", "64"],
                       input="".join(json.dumps(s) + "\n" for s in steps), capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    assert [l for l in r.stdout.splitlines() if l.startswith("done")] == [f"done {i}" for i in range(6)]
    wa, wb = O.forward(cfg, W, a), O.forward(cfg, W, b)
    import numpy as np
    rd = lambda i: torch.from_numpy(np.fromfile(os.path.join(out, f"{i}.f32"), dtype="<f4").reshape(-1, cfg["vocab"]).copy())
    close(rd(0), wa[[0, 14]], 5e-5, "step 0")
    close(rd(1), torch.stack([wa[15], wb[6]]), 5e-5, "step 1")
    for i in range(4):
        close(rd(2 + i), wa[16 + i:17 + i], 5e-5, f"step {2 + i}")
