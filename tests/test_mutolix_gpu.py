"""The Mutolix design on the GPU against the float64 oracle (tests/mutolix_oracle.py): each mechanism alone through the
kernels' bindings, then whole models through the step function, the batch engine and the generation engine."""
import json
import os

import pytest
import torch

from tests import mutolix_oracle as O

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
F32, BF16 = torch.float32, torch.bfloat16


@pytest.fixture(scope="module")
def nsq():
    from promptcache_b200 import _native_seq
    _native_seq.load()
    return _native_seq


def dev(t, dtype=F32):
    return t.to(DEV, dtype).contiguous()


def close(got, want, tol, what=""):
    got, want = got.detach().cpu().to(O.F64), want.to(O.F64)
    err = float((got - want).abs().max() / (want.abs().max() + 1e-30))
    assert err <= tol, f"{what}: relative error {err:.3e} > {tol:.1e}"
    return err


def close_rms(got, want, tol, what=""):
    """Root-mean-square difference relative to the root mean square of the values (for bfloat16 runs, whose largest single
    difference depends on where a rounding happens to be amplified)."""
    got, want = got.detach().cpu().to(O.F64), want.detach().cpu().to(O.F64)
    err = float((got - want).pow(2).mean().sqrt() / want.pow(2).mean().sqrt())
    assert err <= tol, f"{what}: relative rms error {err:.3e} > {tol:.1e}"
    return err


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


LAYERS = lambda: [O.mlstm_layer(), O.attn_layer(), O.attn_layer(heads=2, kv_heads=2, dim=8, vdim=8), O.mlstm_layer(heads=1, dim=16, vdim=8, ff=24)]


# ---- mechanisms alone ---------------------------------------------------------------------------------------------
@pytest.mark.parametrize("width", [40, 257])
def test_rmsnorm_and_gated_output_norm(nsq, width):
    torch.manual_seed(1)
    T, eps = 5, 1e-5
    x, y, g = torch.randn(T, width, dtype=O.F64) * 3, torch.randn(T, width, dtype=O.F64), torch.randn(T, width, dtype=O.F64)
    w, ls, nw = (torch.randn(width, dtype=O.F64) for _ in range(3))
    h = torch.empty(T, width, device=DEV)
    nsq.rmsnorm(dev(x), dev(w), h, eps)
    close(h, O.rms(x, eps, w), 2e-6, "rmsnorm")
    rows = torch.tensor([3, 0], dtype=torch.int32, device=DEV)
    h2 = torch.empty(2, width, device=DEV)
    nsq.rmsnorm(dev(x), dev(w), h2, eps, rows=rows)
    close(h2, O.rms(x[[3, 0]], eps, w), 2e-6, "rmsnorm rows")
    xd, hn = dev(x), torch.empty(T, width, device=DEV)
    nsq.gate_norm_add(xd, dev(y), dev(g), dev(w), dev(ls), eps, dev(nw), hn)
    want = x + O.rms(y * torch.sigmoid(g), eps, w) * ls
    close(xd, want, 2e-6, "gated output norm")
    close(hn, O.rms(want, eps, nw), 4e-6, "next norm")
    xd = dev(x)
    nsq.gate_norm_add(xd, dev(y), None, dev(w), None, eps)   # no gate, no layer scale
    close(xd, x + O.rms(y, eps, w), 2e-6, "plain output norm")


def test_xielu(nsq):
    z = torch.linspace(-6, 6, 97, dtype=O.F64).repeat(3, 1)
    for a in ([0.3, -0.7], [-2.0, 1.5]):
        out = torch.empty(3, 97, device=DEV)
        nsq.xielu(dev(z), out, torch.tensor(a, device=DEV))
        close(out, O.xielu(z, *a), 2e-6, "xielu")


def test_embed_scale(nsq):
    table = torch.randn(11, 24, dtype=O.F64)
    ids = torch.tensor([3, 10, 0, 3], device=DEV)
    out = torch.empty(4, 24, device=DEV)
    nsq.embed(dev(table), ids, out, 0.375)
    close(out, table[ids.cpu()] * 0.375, 1e-7, "embedding")


def _attn_case(nsq, H, G, D, V, lens_pos0, scale, bias=True, sink=True, dtype=F32, seed=0, boost=None, cap=None, split=False, impl=0):
    """Run qk-free attention over hand-made pools: entry b holds pos0[b] rows and brings lens[b] new tokens."""
    g = torch.Generator().manual_seed(seed)
    rnd = lambda *s: torch.randn(*s, generator=g, dtype=O.F64)
    B = len(lens_pos0)
    cap = cap or ((max(p + n for n, p in lens_pos0) + 127) // 128) * 128
    slots = list(range(B))[::-1]  # not the identity
    kp, vp = torch.zeros(B, G, cap, D, dtype=O.F64), torch.zeros(B, G, cap, V, dtype=O.F64)
    qs, want = [], []
    for b, (n, p0) in enumerate(lens_pos0):
        k, v, q = rnd(p0 + n, G, D), rnd(p0 + n, G, V), rnd(n, H, D)
        if boost is not None:      # one key far back is made to stand out for the last query
            j, amount = boost
            q[-1] *= amount
            k[j] = q[-1].view(G, H // G, D).mean(1) / amount * 3
        if dtype == BF16:
            k, v, q = (t.to(BF16).to(O.F64) for t in (k, v, q))
        kp[slots[b], :, :p0 + n] = k.transpose(0, 1)
        vp[slots[b], :, :p0 + n] = v.transpose(0, 1)
        qs.append(q)
        r1 = torch.linspace(0.2, 0.9, H, dtype=O.F64) if bias else None
        r2 = torch.linspace(1.1, 0.3, H, dtype=O.F64) if bias else None
        want.append(O.sink_attention(q, k, v, torch.arange(p0, p0 + n), torch.arange(p0 + n), scale, r1, r2, sink).reshape(n, H * V))
    batch = nsq.Batch(slots, [p for _, p in lens_pos0], [n for n, _ in lens_pos0], torch.device(DEV))
    q = torch.cat(qs).reshape(-1, H * D)
    out = torch.empty(q.shape[0], H * V, device=DEV, dtype=dtype)
    extra = dict(max_keys=cap, workspace=nsq.attn_workspace(q.shape[0], H, V, DEV)) if split else {}
    nsq.attention(dev(q, dtype), dev(kp, dtype), dev(vp, dtype), out, H, scale, dev(r1) if bias else None, dev(r2) if bias else None, sink, batch,
                  impl=impl, **extra)
    return out, torch.cat(want)


@pytest.mark.parametrize("H,G,D,V", [(4, 2, 16, 8), (3, 3, 24, 40), (6, 1, 8, 16), (2, 2, 128, 128)])
def test_attention_shapes_bias_sink(nsq, H, G, D, V):
    for bias, sink in ((True, True), (False, True), (True, False), (False, False)):
        out, want = _attn_case(nsq, H, G, D, V, [(7, 0), (1, 130), (5, 126), (1, 0)], D ** -0.5, bias, sink)
        close(out, want, 5e-6, f"attention bias={bias} sink={sink}")


def test_attention_key_tile_edges_and_far_keys(nsq):
    """Sequences that end just inside and just outside the kernels' key tiles (64, 128), in prompts and in decoding, and
    a far key that dominates the last query."""
    for n_keys in (63, 64, 65, 127, 128, 129, 255, 256, 257, 300):
        out, want = _attn_case(nsq, 4, 2, 16, 8, [(n_keys, 0), (1, n_keys - 1), (2, n_keys - 2)], 0.25, seed=n_keys)
        close(out, want, 5e-6, f"{n_keys} keys")
    for far in (0, 1, 127, 128, 400):
        out, want = _attn_case(nsq, 4, 2, 16, 8, [(1, 700)], 0.5, bias=False, boost=(far, 4.0), seed=far)
        close(out, want, 1e-5, f"far key {far}")
        out, want = _attn_case(nsq, 4, 2, 16, 8, [(701, 0)], 0.5, bias=False, boost=(far, 4.0), seed=far)
        close(out[-1:], want[-1:], 1e-5, f"far key {far} in a prompt")


def test_attention_split_keys(nsq):
    """Decoding over many keys runs as several splits of the keys (whole tiles each) merged by a second launch: sequences of
    unequal lengths in one launch, one of them shorter than a split, with and without the sink and the bias."""
    for bias, sink in ((True, True), (False, False)):
        out, want = _attn_case(nsq, 4, 2, 16, 24, [(1, 2047), (1, 3), (1, 1300), (1, 0)], 0.25, bias, sink, cap=2048, split=True)
        close(out, want, 5e-6, f"split keys bias={bias} sink={sink}")
    out, want = _attn_case(nsq, 2, 1, 16, 8, [(1, 1500)], 0.5, bias=False, boost=(2, 4.0), cap=2048, split=True)
    close(out, want, 1e-5, "far key in the first split")


def test_attention_sink_matters(nsq):
    """With small scores the sink carries a large share of the weight: leaving it out must show."""
    with_sink, want = _attn_case(nsq, 2, 1, 8, 8, [(3, 0)], 0.01)
    without, _ = _attn_case(nsq, 2, 1, 8, 8, [(3, 0)], 0.01, sink=False)
    close(with_sink, want, 5e-6)
    assert float((with_sink - without).abs().max()) > 0.05


def test_attention_bf16_inputs(nsq):
    out, want = _attn_case(nsq, 8, 2, 64, 32, [(200, 0), (1, 333), (40, 100)], 0.125, dtype=BF16)
    close(out, want, 1e-2, "bf16 attention")      # the output is rounded to bfloat16; scores and weights are not


@pytest.mark.parametrize("H,G,D,V", [(4, 2, 96, 32), (2, 2, 64, 64), (4, 1, 128, 128), (2, 1, 256, 256), (3, 3, 24, 40), (2, 1, 8, 200)])
def test_attention_tensor_core_prompts(nsq, H, G, D, V):
    """Prompts in bfloat16 run on the tensor-core kernel: portions that start inside a sequence, ends just inside and just
    outside the 64-row and 64-key tiles, against the oracle and against the plain kernel on the same inputs."""
    for case in ([(64, 0), (65, 63), (17, 0)], [(200, 0), (1, 333), (40, 100)], [(63, 1), (129, 127), (16, 48)]):
        for bias, sink in ((True, True), (False, False)):
            out, want = _attn_case(nsq, H, G, D, V, case, D ** -0.5, bias, sink, dtype=BF16, seed=D + V)
            plain, _ = _attn_case(nsq, H, G, D, V, case, D ** -0.5, bias, sink, dtype=BF16, seed=D + V, impl=1)
            close(out, want, 1e-2, f"tensor-core attention {case} bias={bias} sink={sink}")
            close(out.float(), plain.float().cpu(), 1e-2, "tensor-core vs plain kernel")
            assert float((out.float() - plain.float()).abs().mean()) < 1e-3 * float(plain.float().abs().mean())
    out, want = _attn_case(nsq, H, G, D, V, [(701, 0)], 0.5, bias=False, dtype=BF16, boost=(3, 4.0), seed=1)
    close(out[-1:], want[-1:], 1e-2, "far key in a prompt")


@pytest.mark.parametrize("every", [0, 4])
def test_qk_prep_norm_temperature_mixing_append(nsq, every):
    torch.manual_seed(3)
    H, G, D, V, eps, T, cap = 4, 2, 8, 12, 1e-5, 6, 128
    nq, nk, nv = H * D, G * D, G * V
    qkv = torch.randn(T, nq + nk + nv + 5, dtype=O.F64)
    qw, kw = torch.randn(nq, dtype=O.F64), torch.randn(nk, dtype=O.F64)
    lam = 0.3125
    pos0, slot = 9, 1
    batch = nsq.Batch([slot], [pos0], [T], torch.device(DEV))
    kp, vp, vf = torch.zeros(2, G, cap, D, device=DEV), torch.zeros(2, G, cap, V, device=DEV), torch.randn(2, G, cap, V, device=DEV)
    q_out = torch.empty(T, nq, device=DEV)
    nsq.qk_prep(dev(qkv), (0, nq, nq + nk), dev(qw), dev(kw), eps, H, G, D, V, 0.4, every, q_out, kp, vp, vf, torch.tensor([lam], device=DEV), batch)
    pos = torch.arange(pos0, pos0 + T)
    temp = 1 + 0.4 * torch.log(torch.floor((pos + 1) / every).to(O.F64) + 1) if every else torch.ones(T, dtype=O.F64)
    close(q_out, O.rms(qkv[:, :nq], eps, qw) * temp[:, None], 3e-6, "q")
    close(kp[slot, :, pos0:pos0 + T].transpose(0, 1).reshape(T, nk), O.rms(qkv[:, nq:nq + nk], eps, kw), 3e-6, "k rows")
    first = vf[slot, :, pos0:pos0 + T].transpose(0, 1).reshape(T, nv).cpu().to(O.F64)
    close(vp[slot, :, pos0:pos0 + T].transpose(0, 1).reshape(T, nv), (1 - lam) * qkv[:, nq + nk:nq + nk + nv] + lam * first, 3e-6, "mixed v rows")
    assert float(kp[0].abs().max()) == 0 and float(kp[slot, :, :pos0].abs().max()) == 0 and float(kp[slot, :, pos0 + T:].abs().max()) == 0


@pytest.mark.parametrize("H,D,V", [(2, 8, 16), (1, 16, 8), (3, 12, 20), (2, 64, 128), (1, 16, 160), (1, 200, 24), (1, 260, 16)])
def test_mlstm_gates_and_scan(nsq, H, D, V):
    """The recurrence in one piece, in portions through the pooled state, and as single tokens; large gate values reach
    the cap and the running maximum."""
    torch.manual_seed(5)
    W, T, eps, cap = 24, 37, 1e-5, 6.0
    h = torch.randn(T, W, dtype=O.F64)
    w_i, w_f = torch.randn(H, W, dtype=O.F64) * 2, torch.randn(H, W, dtype=O.F64) * 2
    b_i, b_f = torch.randn(H, dtype=O.F64), torch.randn(H, dtype=O.F64) + 2
    ig, fg = torch.empty(T, H, device=DEV), torch.empty(T, H, device=DEV)
    nsq.mlstm_gates(dev(h), dev(w_i), dev(w_f), dev(b_i), dev(b_f), ig, fg, cap)
    ig_o, fg_o = O.mlstm_gates(h, w_i, b_i, w_f, b_f, cap)
    close(ig, ig_o, 3e-6, "input gate")
    close(fg, fg_o, 3e-6, "forget gate")
    assert float(ig_o.abs().max()) > 0.9 * cap           # the cap is active in this test
    proj = torch.randn(T, 2 * H * D + 2 * H * V + 3, dtype=O.F64)
    offs = (0, H * D, 2 * H * D, 2 * H * D + H * V)
    nw = torch.randn(H * V, dtype=O.F64)
    q = (proj[:, :H * D] * D ** -0.5).view(T, H, D)
    k, v = proj[:, offs[1]:offs[2]].reshape(T, H, D), proj[:, offs[2]:offs[3]].reshape(T, H, V)
    o, state = O.mlstm_recurrence(q, k, v, ig_o, fg_o)
    want = O.rms(o, eps).reshape(T, H * V) * nw * torch.sigmoid(proj[:, offs[3]:offs[3] + H * V])
    for cuts, impl in (([T], 0), ([5, 2, 1, 29], 0), ([1] * T, 0), ([T], 1), ([7, 30], 1)):   # impl 1: the state in shared memory
        s, n, m = torch.full((3, H, D, V), 7.0, device=DEV), torch.full((3, H, D), 7.0, device=DEV), torch.full((3, H), 7.0, device=DEV)
        out, lo = torch.empty(T, H * V, device=DEV), 0
        for c in cuts:          # slot 2 is dirty: a sequence that holds no tokens must start from zero all the same
            batch = nsq.Batch([2], [lo], [c], torch.device(DEV))
            nsq.mlstm_scan(dev(proj[lo:lo + c]), offs, ig[lo:lo + c].contiguous(), fg[lo:lo + c].contiguous(), dev(nw), out[lo:lo + c], s, n, m, eps, batch,
                           impl=impl)
            lo += c
        close(out, want, 2e-5, f"scan cut {cuts[:4]}")
        close(s[2], state[0], 2e-5, "S")
        close(n[2], state[1], 2e-5, "n")
        close(m[2], state[2], 1e-6, "m")
        assert float(s[0].min()) == 7.0  # other slots untouched


@pytest.mark.parametrize("dtype,tol", [(F32, 2e-6), (BF16, 6e-3)])
@pytest.mark.parametrize("M,N,K", [(1, 7, 8), (2, 33, 520), (3, 64, 1024), (5, 10, 264), (8, 129, 96), (9, 12, 64)])
def test_linear_of_few_rows(nsq, dtype, tol, M, N, K):
    """One to eight rows through the weight-streaming kernel (feature counts that are not a multiple of a block's eight, K that
    is not a multiple of a block's pass, a strided input); nine rows take the library product.  Sums are 32-bit in both types."""
    torch.manual_seed(M * N + K)
    x = torch.randn(M, K + 16).to(dtype)
    w, b = (torch.randn(N, K) / K ** 0.5).to(dtype), torch.randn(N).to(dtype)
    for bias in (b, None):
        got = nsq.linear(x.to(DEV)[:, 8:8 + K] if dtype == BF16 else x.to(DEV)[:, 4:4 + K], w.to(DEV), bias.to(DEV) if bias is not None else None,
                         kernel=True)
        xs = x[:, 8:8 + K] if dtype == BF16 else x[:, 4:4 + K]
        want = xs.to(O.F64) @ w.to(O.F64).T + (bias.to(O.F64) if bias is not None else 0)
        close(got, want, tol, f"linear {M}x{N}x{K}")


@pytest.mark.parametrize("H,D,V,cuts", [
    (2, 16, 8, [64]), (1, 32, 40, [63, 65]), (2, 64, 64, [130, 1, 1, 70]), (1, 48, 24, [24, 200]), (1, 256, 72, [129]), (3, 128, 32, [64, 64, 5, 100]),
])
def test_mlstm_chunkwise_bf16(nsq, H, D, V, cuts):
    """The chunkwise tensor-core form (bfloat16 projections, steps of 24 tokens and more) against the token-by-token
    oracle on the SAME bfloat16-rounded projections: chunk edges at 63 / 64 / 65 tokens, steps that continue a pooled state
    (also one left by single-token steps), gates that reach the cap, a dirty slot, and the state it leaves behind.  The
    32-bit factors enter the tensor cores as hi + lo pairs, so the result is 32-bit accurate, far inside bfloat16 rounding."""
    torch.manual_seed(D + V)
    T, eps = sum(cuts), 1e-5
    proj = (torch.randn(T, 2 * H * D + 2 * H * V + 8) * 0.5).to(BF16)
    offs = (0, H * D, 2 * H * D, 2 * H * D + H * V)
    ig_o = (torch.randn(T, H, dtype=O.F64) * 3).clamp(-6, 6)
    fg_o = -torch.rand(T, H, dtype=O.F64) * 0.3
    fg_o[T // 3] = -5.0   # one token nearly wipes the state
    nw = torch.randn(H * V).to(BF16)
    p64 = proj.to(O.F64)
    q = (p64[:, :H * D] * D ** -0.5).view(T, H, D)
    k, v = p64[:, offs[1]:offs[2]].reshape(T, H, D), p64[:, offs[2]:offs[3]].reshape(T, H, V)
    o, state = O.mlstm_recurrence(q, k, v, ig_o, fg_o)
    want = O.rms(o, eps).reshape(T, H * V) * nw.to(O.F64) * torch.sigmoid(p64[:, offs[3]:offs[3] + H * V])
    ig, fg = dev(ig_o), dev(fg_o)
    for impl in (0, 2):   # 2: never the chunkwise kernel (the same inputs token by token)
        s, n, m = torch.full((2, H, D, V), 7.0, device=DEV), torch.full((2, H, D), 7.0, device=DEV), torch.full((2, H), 7.0, device=DEV)
        out, lo = torch.empty(T, H * V, device=DEV, dtype=BF16), 0
        for c in cuts:
            batch = nsq.Batch([1], [lo], [c], torch.device(DEV))
            nsq.mlstm_scan(proj[lo:lo + c].to(DEV), offs, ig[lo:lo + c].contiguous(), fg[lo:lo + c].contiguous(), nw.to(DEV), out[lo:lo + c], s, n, m,
                           eps, batch, impl=impl)
            lo += c
        close(s[1], state[0], 3e-5, f"S (impl {impl})")
        close(n[1], state[1], 3e-5, f"n (impl {impl})")
        close(m[1], state[2], 1e-6, f"m (impl {impl})")
        close(out, want, 6e-3, f"output (impl {impl})")   # the output itself is rounded to bfloat16
        assert float(s[0].min()) == 7.0


@pytest.mark.parametrize("H,D,V,lens,pos0,slots", [
    (2, 32, 48, [100, 3, 64], [0, 40, 9], [2, 0, 1]),
    # enough blocks for the 32-column slices (few blocks take 16-column slices)
    (8, 16, 72, [30, 65, 24, 5, 40, 33, 64, 70, 26, 31], [0, 3, 0, 9, 1, 0, 0, 7, 2, 0], [9, 0, 8, 1, 7, 2, 6, 3, 5, 4]),
])
def test_mlstm_chunkwise_batch_of_unequal_entries(nsq, H, D, V, lens, pos0, slots):
    """Entries of unequal lengths in one launch, some continuing pooled states: each equals the entry alone, token by token."""
    torch.manual_seed(3)
    eps = 1e-5
    T = sum(lens)
    proj = (torch.randn(T, 2 * H * D + 2 * H * V) * 0.5).to(BF16).to(DEV)
    offs = (0, H * D, 2 * H * D, 2 * H * D + H * V)
    ig, fg = torch.randn(T, H, device=DEV), -torch.rand(T, H, device=DEV) * 0.2
    nw = torch.randn(H * V).to(BF16).to(DEV)
    ns = len(lens)
    s0, n0, m0 = torch.randn(ns, H, D, V, device=DEV), torch.randn(ns, H, D, device=DEV), torch.rand(ns, H, device=DEV)
    s, n, m = s0.clone(), n0.clone(), m0.clone()
    out = torch.empty(T, H * V, device=DEV, dtype=BF16)
    nsq.mlstm_scan(proj, offs, ig, fg, nw, out, s, n, m, eps, nsq.Batch(slots, pos0, lens, torch.device(DEV)))
    lo = 0
    for b, c in enumerate(lens):
        s1, n1, m1 = s0.clone(), n0.clone(), m0.clone()
        o1 = torch.empty(c, H * V, device=DEV, dtype=BF16)
        nsq.mlstm_scan(proj[lo:lo + c], offs, ig[lo:lo + c].contiguous(), fg[lo:lo + c].contiguous(), nw, o1, s1, n1, m1, eps,
                       nsq.Batch([slots[b]], [pos0[b]], [c], torch.device(DEV)), impl=2)
        close(out[lo:lo + c], o1.cpu(), 6e-3, f"entry {b}")
        close(s[slots[b]], s1[slots[b]].cpu(), 3e-5, f"state of entry {b}")
        close(n[slots[b]], n1[slots[b]].cpu(), 3e-5, f"n of entry {b}")
        lo += c


# ---- whole models (float32 rounding accumulates over the layers: 1e-4 of the largest value) ---------------------------
def test_whole_prompt_fp32_layers_and_logits(tmp_path):
    cfg, W = O.random_model(LAYERS(), width=40, vocab=61, seed=1)
    m = load(tmp_path, cfg, W)
    toks = tokens(45, 61, 0)
    m.layer_trace = []
    seq = m.new_sequence()
    got = m.step([(seq, toks)], [list(range(45))])
    ref_layers = []
    want = O.forward(cfg, W, toks, ref_layers)
    for i, (a, b) in enumerate(zip(m.layer_trace, ref_layers)):
        close(a, b, 1e-4, f"residual stream after layer {i}")
    close(got, want, 1e-4, "logits")


@pytest.mark.parametrize("layers,width,vocab", [
    ([O.attn_layer(heads=2, kv_heads=1, dim=8, vdim=24, ff=None), O.mlstm_layer(heads=3, dim=8, vdim=12, ff=20), O.attn_layer(heads=2, kv_heads=1, dim=8, vdim=24, every=0)], 36, 50),
    ([O.mlstm_layer(heads=1, dim=8, vdim=8)], 24, 30),
    ([O.attn_layer(heads=1, kv_heads=1, dim=32, vdim=16, v_mix=False, every=1), O.attn_layer(heads=4, kv_heads=4, dim=8, vdim=8, v_mix=True), O.attn_layer(heads=4, kv_heads=4, dim=16, vdim=8, v_mix=True)], 72, 33),
])
def test_other_sizes_and_orders(tmp_path, layers, width, vocab):
    cfg, W = O.random_model(layers, width=width, vocab=vocab, seed=2, emb_scale=1.0)
    m = load(tmp_path, cfg, W)
    toks = tokens(21, vocab, 4)
    seq = m.new_sequence()
    got = m.step([(seq, toks)], [list(range(21))])
    close(got, O.forward(cfg, W, toks), 1e-4, "logits")


def test_portions_decode_and_graph_replay(tmp_path):
    """Whole prompt = portions of 2..many tokens = token by token (eager and through the replayed decode graph); the
    query temperature steps every 8 positions and the prompt crosses key tiles."""
    cfg, W = O.random_model(LAYERS(), seed=3)
    m = load(tmp_path, cfg, W)
    n = 150
    toks = tokens(n, 61, 7)
    want = O.forward(cfg, W, toks)
    for cuts in ([n], [2, 2, 3, 60, 1, 2, 80], [128, 1, 21], [127, 2, 21]):
        seq, lo, rows = m.new_sequence(), 0, []
        for c in cuts:
            rows.append(m.step([(seq, toks[lo:lo + c])], [list(range(c))]))
            lo += c
        close(torch.cat(rows), want, 1e-4, f"portions {cuts}")
        seq.free()
    for graphs in (False, True):
        m.use_cuda_graphs = graphs
        seq = m.new_sequence()
        rows = [m.step([(seq, toks[:100])], [list(range(100))])]
        rows += [m.step([(seq, [t])]) for t in toks[100:]]
        close(torch.cat(rows), want, 1e-4, f"decode graphs={graphs}")
        seq.free()
    assert any(k[0] == 1 for k in m._graphs)      # the decode graph was captured and replayed


def test_batches_of_unequal_requests_and_slot_reuse(tmp_path):
    cfg, W = O.random_model(LAYERS(), seed=4)
    m = load(tmp_path, cfg, W)
    from promptcache_b200.batch_engine import BatchEngine
    eng = BatchEngine(m, max_tokens=700)
    prompts = [tokens(n, 61, 10 + n) for n in (1, 37, 130, 5)]
    wants = [O.forward(cfg, W, p) for p in prompts]
    # prompts together (all but their last 3 tokens), then decoded together; shorter requests end earlier
    got = eng.step([(f"r{i}", p[:max(1, len(p) - 3)], None) for i, p in enumerate(prompts)], end=["r0"])
    for i, p in enumerate(prompts):
        close(got[i], wants[i][max(1, len(p) - 3) - 1], 1e-4, f"prefill of request {i} in a batch")
    for step in range(3):
        live = [i for i, p in enumerate(prompts) if len(p) > 3]
        got = eng.step([(f"r{i}", [prompts[i][len(prompts[i]) - 3 + step]], [0]) for i in live])
        for j, i in enumerate(live):
            close(got[j], wants[i][len(prompts[i]) - 3 + step], 1e-4, f"decode step {step} of request {i} in a batch")
    used = {s.slot for s in eng.live.values()}
    for i in (1, 2, 3):
        eng.end(f"r{i}")
    assert not eng.live and not m.pool.rows
    # the freed slots are used again by other requests, longer and shorter than their previous owners
    again = [tokens(n, 61, 50 + n) for n in (90, 3, 140)]
    got = eng.step([(f"s{i}", p, list(range(len(p)))) for i, p in enumerate(again)])
    assert {s.slot for s in eng.live.values()} <= used | {0, 1, 2, 3}
    lo = 0
    for p in again:
        close(got[lo:lo + len(p)], O.forward(cfg, W, p), 1e-4, "request in a reused slot")
        lo += len(p)
    with pytest.raises(ValueError):
        eng.step([("big", tokens(600, 61, 1), None)])   # over the token budget


def test_long_decoding_with_pool_growth(tmp_path):
    cfg, W = O.random_model([O.attn_layer(every=16), O.mlstm_layer(), O.attn_layer(every=16)], seed=5)
    m = load(tmp_path, cfg, W)
    toks = tokens(300, 61, 9)
    want = O.forward(cfg, W, toks)
    a, b = m.new_sequence(), m.new_sequence()
    rows = [m.step([(a, toks[:3]), (b, toks[:120])], [[0, 1, 2], [119]])[:3]]
    for t in range(3, 300):                  # a grows past the pool's first capacity while b stays live
        rows.append(m.step([(a, [toks[t]])]))
    close(torch.cat(rows), want, 1e-4, "300 tokens, 297 of them decoded")
    close(m.step([(b, toks[120:130])])[0], want[129], 1e-4, "the sequence that waited")


def test_bf16_model_is_close_and_cut_invariant(tmp_path):
    cfg, W = O.random_model(LAYERS(), seed=6)
    m = load(tmp_path, cfg, W, dtype=BF16)
    toks = tokens(140, 61, 3)
    want = O.forward(cfg, W, toks)
    seq = m.new_sequence()
    whole = m.step([(seq, toks)], [list(range(140))])
    e1 = close_rms(whole, want, 8e-2, "bf16 logits")
    seq2, other = m.new_sequence(), m.new_sequence()
    part = [m.step([(seq2, toks[:129]), (other, toks[5:50])], [list(range(129)), []])]
    part += [m.step([(seq2, [t]), (other, [7])], [[0], []]) for t in toks[129:]]
    e2 = close_rms(torch.cat(part), whole, 8e-2, "bf16: cut and batched vs whole")
    print(f"bf16 relative rms: vs oracle {e1:.3e}, cut vs whole {e2:.3e}")


def test_greedy_generation_through_the_engines(tmp_path):
    from promptcache_b200 import GenerationEngine, GenerationParameters
    from promptcache_b200.batch_engine import BatchEngine
    from promptcache_b200.model import Mutolix
    cfg, W = O.random_model(LAYERS(), seed=8)
    m = load(tmp_path, cfg, W)
    lm = Mutolix("tiny", model=m)
    prompts = [tokens(n, 61, 20 + n) for n in (9, 33, 2)]
    wants = [O.greedy(cfg, W, p, 6) for p in prompts]
    params = GenerationParameters(temperature=0.0, max_new_tokens=6, stop_token_ids=[], stop_str=[])
    for p, w in zip(prompts, wants):
        outs = list(GenerationEngine(lm).generate(p, list(range(len(p))), params, None, stream_interval=2))
        assert outs[-1].new_text == lm.decode(w)
    assert not m.pool.rows                                   # the engines gave their slots back
    assert BatchEngine(m).generate(prompts, params) == wants
    stop = wants[1][2]
    stopped = BatchEngine(m, max_tokens=64).generate(prompts, GenerationParameters(temperature=0.0, max_new_tokens=6, stop_token_ids=[stop]))
    assert stopped[1] == wants[1][:wants[1].index(stop) + 1]


def test_trace_replay_command(tmp_path):
    """bin/trace_run end to end: a prompt step with wanted places, a step that wants nothing, a decode step, `end`."""
    import subprocess
    import numpy as np
    cfg, W = O.random_model(LAYERS(), seed=9)
    folder = str(tmp_path / "ckpt")
    write_checkpoint(folder, cfg, W)
    toks = tokens(12, 61, 2)
    want = O.forward(cfg, W, toks)
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": toks[:10], "want": [0, 9]}], "end": []},
             {"step": 1, "entries": [{"id": "a", "tokens": toks[10:11], "want": []}], "end": []},
             {"step": 2, "entries": [{"id": "a", "tokens": toks[11:], "want": [0]}, {"id": "b", "tokens": toks[:4], "want": [3]}], "end": ["a", "b"]}]
    out = str(tmp_path / "out")
    r = subprocess.run([os.path.join(root, "bin", "trace_run"), "--model", folder, "--dtype", "float32", "--out", out, "--max-tokens", "64"],
                       input="".join(json.dumps(s) + "\n" for s in steps), capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    assert [l for l in r.stdout.splitlines() if l.startswith("done")] == ["done 0", "done 1", "done 2"]
    assert not os.path.exists(os.path.join(out, "1.f32"))
    s0 = torch.from_numpy(np.fromfile(os.path.join(out, "0.f32"), dtype="<f4").reshape(2, 61))
    s2 = torch.from_numpy(np.fromfile(os.path.join(out, "2.f32"), dtype="<f4").reshape(2, 61))
    close(s0, want[[0, 9]], 1e-4)
    close(s2, torch.stack([want[11], want[3]]), 1e-4)
