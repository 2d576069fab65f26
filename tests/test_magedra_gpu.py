"""The Magedra decoder in the engine against the plain statement of its equations.

Kernels and parts alone; the stream after every layer; whole prompts; token-by-token decoding; portions
down to two tokens; unequal requests in one batch against each alone; rows, pages and state slots that are
used again; a planted key that decides an attention output, far back, at page borders, on either side of a
chunk of 128 keys and of a window's edge, in prompts and decoded; a planted write that a recurrent state must
carry over hundreds of tokens; long decoding; greedy generation through the engine's entry point and
scheduler; the command line; a replay through bin/trace_run.
"""

import json

import numpy as np
import pytest
import torch

import plain_magedra as plain
from bofusun_tiny import Harness, rel_err
from magedra_tiny import TINY, make_folder, save_weights
from traces import Trace, compare, last_decoded, mixed, portions, run_trace, whole

pytestmark = pytest.mark.gpu
DEV = "cuda"
TOL = {torch.float32: 2e-4, torch.bfloat16: 6e-2}
PART_TOL = {torch.float32: 1e-4, torch.bfloat16: 4e-2}
DTYPES = [torch.float32, torch.bfloat16]
F64 = torch.float64


def tokens(vocab, n, seed):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (n,), generator=g).tolist()


def i32(x):
    return torch.tensor(x, dtype=torch.int32, device=DEV)


def part_err(got, want):
    return float((got - want).abs().max() / want.abs().max())


# ------------------------------------------------------------------------------------------
# kernels alone

@pytest.mark.parametrize("s,d", [(1, 40), (3, 36), (4, 200), (8, 130)])
@pytest.mark.parametrize("center", [True, False])
def test_streams_fold_and_norm(s, d, center):
    """The folding kernel against the equations: streams that start as copies, a branch of several partial sums
    with a bias, two branches side by side, rows that are only read (a row index), the reading itself."""
    from socrates_b200.kernels import ops
    g = torch.Generator().manual_seed(s * d)
    N, eps, mult = 9, 1e-5, 0.7
    init = torch.randn(N, d, generator=g)
    mix, out_w, in_w = torch.rand(s, s, generator=g) - 0.2, torch.rand(s, generator=g) + 0.3, torch.rand(s, generator=g) + 0.1
    gain = 1 + 0.1 * torch.randn(d, generator=g)
    a, b, bias = torch.randn(3, N, d, generator=g), torch.randn(2, N, d, generator=g), torch.randn(d, generator=g)

    def norm(u):
        u = u.double()
        return plain.layer_norm(u, gain.double(), eps) if center else plain.rms_norm(u, gain.double(), eps)

    xs = init.double()[None].repeat(s, 1, 1)                                  # [s, N, d]
    streams = torch.zeros(N, s, d, device=DEV)
    out = torch.empty(N, d, device=DEV)
    # 1. the streams are made from the embedding's output and read
    ops.hyper_fold_norm(streams, init.to(DEV), None, 1.0, None, 1.0, None, None, None, 1.0, in_w.to(DEV), gain.to(DEV),
                        eps, center, out)
    assert part_err(out.double().cpu(), norm(torch.einsum("s,snd->nd", in_w.double(), xs))) < 1e-5
    assert torch.equal(streams.cpu(), init[:, None, :].repeat(1, s, 1))
    # 2. a branch with a bias joins; 3. two branches side by side, each with its scale
    for second in (None, b):
        y = 1.3 * (a.double().sum(0) + bias.double()) + (0.6 * second.double().sum(0) if second is not None else 0)
        xs = torch.einsum("st,snd->tnd", mix.double(), xs) + mult * out_w.double()[:, None, None] * y[None]
        ops.hyper_fold_norm(streams, None, a.to(DEV), 1.3, second.to(DEV) if second is not None else None, 0.6,
                            bias.to(DEV), mix.to(DEV), out_w.to(DEV), mult, in_w.to(DEV), gain.to(DEV), eps, center, out)
        assert part_err(out.double().cpu(), norm(torch.einsum("s,snd->nd", in_w.double(), xs))) < 1e-5
        assert part_err(streams.double().cpu(), xs.permute(1, 0, 2)) < 1e-5
    # 4. a few rows only, the plain sum, nothing written; the reading itself
    before = streams.clone()
    idx = [7, 2, 2, 0]
    y = a.double().sum(0)
    xs2 = torch.einsum("st,snd->tnd", mix.double(), xs) + mult * out_w.double()[:, None, None] * y[None]
    few, read = torch.empty(4, d, device=DEV, dtype=torch.bfloat16), torch.empty(4, d, device=DEV)
    ops.hyper_fold_norm(streams, None, a.to(DEV), 1.0, None, 1.0, None, mix.to(DEV), out_w.to(DEV), mult, None,
                        gain.to(DEV), eps, center, few, i32(idx), read)
    assert part_err(read.double().cpu(), xs2.sum(0)[idx]) < 1e-5
    assert part_err(few.double().cpu(), norm(xs2.sum(0))[idx]) < 1e-2
    assert torch.equal(streams, before)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("W", [11, 130, 224])
def test_min_gru_kernel(dtype, W):
    """Two requests, one continued from a state, in one launch."""
    from socrates_b200.kernels import ops
    g = torch.Generator().manual_seed(W)
    lens = [37, 5]
    proj = (torch.randn(sum(lens), 3 * W + 3, generator=g) * 2).to(dtype)
    bz, bx = torch.randn(W, generator=g), torch.randn(W, generator=g)
    state = torch.zeros(4, W)
    state[2] = torch.randn(W, generator=g)
    want, at = [], 0
    for r, n in enumerate(lens):
        p = proj[at:at + n].double()
        z = plain.sigmoid(p[:, :W] + bz.double())
        u = p[:, W:2 * W] + bx.double()
        c = torch.where(u >= 0, u + 0.5, plain.sigmoid(u))
        S = state[[3, 2][r]].double()
        for t in range(n):
            S = (1 - z[t]) * S + z[t] * c[t]
            want.append(S * plain.silu(p[t, 2 * W:3 * W]))
        at += n
    out = torch.empty(sum(lens), W, device=DEV, dtype=dtype)
    st = state.to(DEV)
    ops.min_gru(out, proj.to(DEV), bz.to(DEV), bx.to(DEV), st, i32([0, 37, 42]), i32([3, 2]))
    assert part_err(out.double().cpu(), torch.stack(want)) < (2e-6 if dtype == torch.float32 else 1e-2)
    assert part_err(st[2].double().cpu(), S) < 1e-5 and torch.equal(st[[0, 1]].cpu(), state[[0, 1]])


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("shape", [(2, 12, 20), (1, 70, 9), (3, 130, 8), (2, 5, 7), (4, 48, 64)])
@pytest.mark.parametrize("lens", [[45, 3], [300, 40], [1, 1]])
def test_gated_linear_attention_kernel(dtype, shape, lens):
    """Two requests, one continued from a state, in one launch; long portions run as segments joined in order."""
    from socrates_b200.kernels import ops
    H, D, Dv = shape
    g = torch.Generator().manual_seed(sum(shape))
    eps = 1e-5
    C = 2 * H * D + H * Dv
    proj = (torch.randn(sum(lens), C, generator=g) * 1.5).to(dtype)
    fb, low = torch.randn(H * D, generator=g) + 1.5, torch.rand(H * D, generator=g) * 0.9
    nw = 1 + 0.1 * torch.randn(Dv, generator=g)
    state = torch.zeros(3, H, D, Dv)
    state[0] = torch.randn(H, D, Dv, generator=g)
    want, at = [], 0
    for r, n in enumerate(lens):
        p = proj[at:at + n].double()
        q = plain.silu(p[:, :H * D]).view(n, H, D)
        f = (low.double() + (1 - low.double()) * plain.sigmoid(p[:, H * D:2 * H * D] + fb.double())).view(n, H, D)
        v = p[:, 2 * H * D:].view(n, H, Dv)
        S = state[[1, 0][r]].double()
        for t in range(n):
            S = f[t][:, :, None] * S + (1 - f[t])[:, :, None] * v[t][:, None, :]
            want.append(plain.rms_norm(torch.einsum("hde,hd->he", S, q[t]), nw.double(), eps).reshape(H * Dv))
        at += n
    out = torch.empty(sum(lens), H * Dv, device=DEV, dtype=dtype)
    st = state.to(DEV)
    need = ops.gated_linear_attention_seg_scratch(2, sum(lens) - 1, H, D, Dv)
    assert (need > 0) == (sum(lens) > 129)
    ops.gated_linear_attention(out, proj.to(DEV), (0, H * D, 2 * H * D), fb.to(DEV), low.to(DEV), nw.to(DEV), st,
                               i32([0, lens[0], sum(lens)]), i32([1, 0]), H, D, Dv, eps,
                               torch.empty(sum(lens) * H * Dv, device=DEV),
                               seg_scratch=torch.empty(need, device=DEV) if need else None)
    assert part_err(out.double().cpu(), torch.stack(want)) < (1e-5 if dtype == torch.float32 else 2e-2)
    assert part_err(st[0].double().cpu(), S) < 1e-5 and torch.equal(st[2].cpu(), state[2])


@pytest.mark.parametrize("dtype", DTYPES)
def test_small_steps(dtype):
    """The clamped gated unit (a matrix and partial sums), the norms of column segments, a matrix per head in both
    directions with carried values, the constant on the logits."""
    from socrates_b200.kernels import ops
    g = torch.Generator().manual_seed(1)
    tol = 1e-5 if dtype == torch.float32 else 1e-2
    for N, F_ in ((13, 21), (9, 24), (300, 64)):           # rows of single values, and of whole 16-byte pieces
        x = (torch.randn(N, 2 * F_, generator=g) * 2).to(dtype)
        bg, bu = torch.randn(F_, generator=g), torch.randn(F_, generator=g)
        for lim in (0.5, 2.0):
            gg = (x.double()[:, :F_] + bg.double()).clamp(max=lim)
            uu = (x.double()[:, F_:] + bu.double()).clamp(-lim, lim)
            want = gg * plain.sigmoid(1.702 * gg) * (uu + 1.0)
            out = torch.empty(N, F_, device=DEV, dtype=dtype)
            ops.glu_clamp(out, x.to(DEV), bg.to(DEV), bu.to(DEV), lim, 1.702, 1.0)
            assert part_err(out.double().cpu(), want) < tol
            parts = torch.stack([x.float() * 0.25, x.float() * 0.75]).to(DEV)
            ops.glu_clamp(out, parts, bg.to(DEV), bu.to(DEV), lim, 1.702, 1.0)
            assert part_err(out.double().cpu(), want) < tol
    N = 13
    # segments
    x = torch.randn(N, 50, generator=g).to(dtype)
    g1, g2 = torch.rand(17, generator=g) + 0.5, torch.rand(20, generator=g) + 0.5
    a, b = torch.zeros(N, 17, device=DEV, dtype=dtype), torch.zeros(N, 60, device=DEV, dtype=dtype)
    ops.segment_norm(x.to(DEV), [(3, 17, g1.to(DEV), [(a, 0)]), (20, 20, g2.to(DEV), [(b, 5), (b, 40)]),
                                 (40, 10, None, [(b, 25)])], 1e-5)
    assert part_err(a.double().cpu(), plain.rms_norm(x.double()[:, 3:20], g1.double(), 1e-5)) < tol
    w2 = plain.rms_norm(x.double()[:, 20:40], g2.double(), 1e-5)
    assert part_err(b.double().cpu()[:, 5:25], w2) < tol and part_err(b.double().cpu()[:, 40:60], w2) < tol
    assert torch.equal(b.cpu()[:, 25:35], x[:, 40:50])
    # a matrix per head
    H, A, B = 3, 7, 150
    w = torch.randn(H * A, B, generator=g).to(dtype)
    for N in (5, 37):
        xa = torch.randn(N, H * (A + 2), generator=g).to(dtype)          # per head [2 carried | A inputs]
        y = torch.zeros(N, H * (B + 2), device=DEV, dtype=dtype)
        ops.head_matmul(y, 2, B + 2, xa.to(DEV), 2, A + 2, w.to(DEV), H, transposed=True, carry=2)
        want = torch.einsum("nha,hab->nhb", xa.double().view(N, H, A + 2)[..., 2:], w.double().view(H, A, B))
        got = y.double().cpu().view(N, H, B + 2)
        assert part_err(got[..., 2:], want) < tol and torch.equal(got[..., :2], xa.double().view(N, H, A + 2)[..., :2])
        xb = torch.randn(N, H * B, generator=g).to(dtype)
        y = torch.zeros(N, H * A, device=DEV, dtype=dtype)
        ops.head_matmul(y, 0, A, xb.to(DEV), 0, B, w.to(DEV), H, transposed=False)
        want = torch.einsum("nhb,hab->nha", xb.double().view(N, H, B), w.double().view(H, A, B))
        assert part_err(y.double().cpu().view(N, H, A), want) < tol
    z = torch.randn(4, 33, generator=g).to(DEV)
    want = z.double().cpu() * 0.37
    ops.scale_(z, 0.37)
    assert part_err(z.double().cpu(), want) < 1e-6


def dense_talking(q, k, v, talk, scale, window):
    """q [n, H, dk], k [n, G, dk], v [n, G, dv] of one request, float64: [n, H, dv]."""
    n, H = q.shape[0], q.shape[1]
    kv_of = torch.arange(H) // (H // k.shape[1])
    s = torch.einsum("hg,gij->hij", talk, torch.einsum("ihd,jhd->hij", q, k[:, kv_of]) * scale)
    i, j = torch.arange(n)[:, None], torch.arange(n)[None, :]
    seen = (j <= i) & ((i - j < window) if window else torch.ones(n, n, dtype=torch.bool))
    p = torch.softmax(s.masked_fill(~seen, float("-inf")), dim=-1)
    return torch.einsum("hij,jhe->ihe", p, v[:, kv_of])


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("shape", [(4, 2, 16, 8), (6, 6, 8, 130), (2, 1, 64, 32), (3, 3, 6, 10), (8, 2, 32, 64), (1, 1, 24, 16)])
@pytest.mark.parametrize("window", [0, 7, 16, 130])
def test_attention_with_mixed_scores(dtype, shape, window):
    """Tiles of prompt portions (the chosen tile size, and tiles of one and of three queries) and decode shares
    against the dense computation, for two requests in scattered pages: a whole prompt, and a portion behind an
    earlier one; with and without the gate."""
    from socrates_b200.kernels import ops
    H, G, dk, dv = shape
    page, scale = 16, 0.3
    g = torch.Generator().manual_seed(sum(shape) + window)
    lens, new = [330, 41], [330, 6]
    order = torch.randperm(25, generator=g).tolist()
    tables = [[1 + o for o in order[:21]], [1 + o for o in order[21:24]] + [0] * 18]
    k_pool, v_pool = torch.zeros(26, G, page, dk, dtype=dtype), torch.zeros(26, G, page, dv, dtype=dtype)
    talk = torch.eye(H) * 0.8 + 0.4 * torch.randn(H, H, generator=g)
    qs, wants = [], []
    for r, n in enumerate(lens):
        q, k, v = (torch.randn(n, h, d, generator=g).to(dtype) for h, d in ((H, dk), (G, dk), (G, dv)))
        for p in range(n):
            k_pool[tables[r][p // page], :, p % page] = k[p]
            v_pool[tables[r][p // page], :, p % page] = v[p]
        o = dense_talking(q.double(), k.double(), v.double(), talk.double(), scale, window)
        qs.append(q[n - new[r]:].reshape(new[r], H * dk))
        wants.append(o[n - new[r]:].reshape(new[r], H * dv))
    q, want = torch.cat(qs).to(DEV).contiguous(), torch.cat(wants)
    N = q.shape[0]
    gate = torch.randn(N, H * dv + 5, generator=g).to(dtype)
    gated = want * plain.sigmoid(gate.double()[:, :H * dv])
    k_pool, v_pool, table, talk = k_pool.to(DEV), v_pool.to(DEV), i32(tables), talk.to(DEV)
    starts, rows, first = i32([0, new[0], N]), i32([0, 1]), i32([lens[0] - new[0], lens[1] - new[1]])
    tol = 2e-5 if dtype == torch.float32 else 2e-2
    assert ops.attention_talk_tile(H, G, dk, dv) >= 1
    for qt in (0, 1, 3):
        out = torch.empty(N, H * dv, device=DEV, dtype=dtype)
        ops.attention_talk(out, q, k_pool, v_pool, table, starts, rows, first, talk, H, scale, window, queries_per_tile=qt)
        assert part_err(out.double().cpu(), want) < tol, qt
    ops.attention_talk(out, q, k_pool, v_pool, table, starts, rows, first, talk, H, scale, window, gate=gate.to(DEV))
    assert part_err(out.double().cpu(), gated) < tol
    # decode: every token a request of its own row; here the same two rows, token by token, in key shares
    for NP in (1, 3, 16):
        po = torch.empty(N * H * NP * dv, device=DEV) if NP > 1 else None
        pm = torch.empty(N * H * NP * 2, device=DEV) if NP > 1 else None
        got = []
        for n in range(N):
            r = 0 if n < new[0] else 1
            pos = (lens[0] - new[0] + n) if r == 0 else (lens[1] - new[1] + n - new[0])
            if n % 37 and n < new[0] - 3:
                continue                                  # a sample of the long request's tokens
            o1 = torch.empty(1, H * dv, device=DEV, dtype=dtype)
            ops.attention_talk(o1, q[n:n + 1], k_pool, v_pool, table, i32([0, 1]), i32([r]), i32([pos]), talk, H, scale,
                               window, gate=gate[n:n + 1].to(DEV), queries_per_tile=1, num_partitions=NP, part_o=po, part_ml=pm)
            got.append((n, o1.double().cpu()[0]))
        for n, o1 in got:
            assert part_err(o1, gated[n]) < tol, (NP, n)


# ------------------------------------------------------------------------------------------
# parts alone

def run_part(h, part, x, dtype, sizes, entry=None):
    """Feed x [n, width] through a mixer (entry: its place in the run order) or a feed-forward in portions."""
    from socrates_b200.engine.context import CacheView
    from socrates_b200.engine.runner import StepEntry
    n = x.shape[0]
    h.cache.assign(1)
    got, start, k = [], 0, 0
    while start < n:
        c = min(sizes[min(k, len(sizes) - 1)], n - start)
        assert h.cache.reserve(1, start + c)
        ctx = h.runner.prepare([StepEntry(1, [0] * c, start, [c - 1])])
        xin = x[start:start + c].to(dtype).to(DEV).contiguous()
        b = part.forward(ctx, xin) if entry is None else part.forward(ctx, xin, CacheView(h.cache, entry, True))
        y = b.scale * (b.partial.sum(0).double() + (b.bias.double() if b.bias is not None else 0))
        if b.also is not None:
            y = y + b.also.scale * b.also.partial.sum(0).double()
        got.append(y.cpu())
        h.cache.commit(1, start + c)
        start, k = start + c, k + 1
    h.cache.release(1)
    return torch.cat(got)


def plain_mixer(kind, x, w, pre, m, eps):
    return plain.mixer(kind, x, w, pre, m, eps, torch.arange(x.shape[0]))


@pytest.mark.parametrize("dtype", DTYPES)
def test_mixers_alone(tmp_path, dtype):
    g = torch.Generator().manual_seed(4)
    for name, layer, entry in (("A", 0, 0), ("A", 0, 4), ("A", 1, 1), ("A", 1, 2), ("A", 2, 3), ("B", 0, 0), ("B", 1, 1),
                               ("B", 2, 2), ("C", 0, 2), ("C", 1, 1), ("D", 0, 3), ("D", 1, 1), ("D", 2, 2), ("E", 0, 0), ("E", 2, 2)):
        folder, cfg, w = make_folder(tmp_path, name)
        spec = [l for l in cfg["layers"] if "weights_of" not in l][layer]
        pre = "l%d.mix." % cfg["layers"].index(spec)
        n = 170 if name in ("C", "E") else 70
        x = (torch.randn(n, cfg["width"], generator=g) * 1.5).bfloat16().double()
        want = plain_mixer(spec["type"], x, w, pre, spec["mixer"], cfg["norm"]["eps"])
        for sizes in ((n,), (1,), (33, 2, 1, 30, 1)):
            h = Harness(folder, dtype, max_len=320)
            got = run_part(h, h.model.layers[layer].mixer, x, dtype, sizes, entry=entry)
            assert part_err(got, want) < PART_TOL[dtype], (name, layer, sizes)


def test_tensor_core_form_of_attention_with_mixed_scores(tmp_path, monkeypatch):
    """One long prompt portion in the bfloat16 engine: keys gathered out of their pages, both products through the
    engine's matrix product, mixing, mask and softmax in between; whole, behind an earlier portion, and in blocks
    of queries; against the plain statement and against the CUDA-core kernel."""
    from socrates_b200.parts.talking_attention import TalkingAttention
    g = torch.Generator().manual_seed(14)
    for name, layer, entry in (("A", 1, 1), ("C", 0, 0), ("E", 0, 0)):
        folder, cfg, w = make_folder(tmp_path, name)
        spec = [l for l in cfg["layers"] if "weights_of" not in l][layer]
        pre = "l%d.mix." % cfg["layers"].index(spec)
        n = 300
        x = (torch.randn(n, cfg["width"], generator=g) * 1.5).bfloat16().double()
        want = plain_mixer(spec["type"], x, w, pre, spec["mixer"], cfg["norm"]["eps"])
        monkeypatch.setattr(TalkingAttention, "DENSE_FROM", 1 << 30)
        h = Harness(folder, torch.bfloat16, max_len=320)
        cores = run_part(h, h.model.layers[layer].mixer, x, torch.bfloat16, (n,), entry=entry)
        assert not any(k[0] == "talk_s" for k in h.runner.buffers._flat)
        for sizes, most in (((n,), 1 << 27), ((70, 230), 1 << 27), ((n,), 64 * 320 * spec["mixer"]["left"]["heads"])):
            monkeypatch.setattr(TalkingAttention, "DENSE_FROM", 128)
            monkeypatch.setattr(TalkingAttention, "DENSE_SCORES", most)
            h = Harness(folder, torch.bfloat16, max_len=320)
            got = run_part(h, h.model.layers[layer].mixer, x, torch.bfloat16, sizes, entry=entry)
            assert any(k[0] == "talk_s" for k in h.runner.buffers._flat), "the tensor-core form did not run"
            assert part_err(got, want) < PART_TOL[torch.bfloat16], (name, sizes)
            assert part_err(got, cores) < PART_TOL[torch.bfloat16], (name, sizes)


@pytest.mark.parametrize("dtype", DTYPES)
def test_feed_forwards_alone(tmp_path, dtype):
    g = torch.Generator().manual_seed(6)
    for name, layer in (("A", 0), ("B", 0), ("C", 1), ("D", 2)):
        folder, cfg, w = make_folder(tmp_path, name)
        spec = [l for l in cfg["layers"] if "weights_of" not in l][layer]
        pre = "l%d.mlp." % cfg["layers"].index(spec)
        x = (torch.randn(50, cfg["width"], generator=g) * 1.5).bfloat16().double()
        want = plain.feed_forward(x, w, pre, spec["mlp"])
        pre_act = x @ w[pre + "gate"].T + w[pre + "gate.b"]
        assert float((pre_act > spec["mlp"]["limit"]).double().mean()) > 0.02      # the clamp bites
        for sizes in ((50,), (1,), (7, 2, 16)):
            h = Harness(folder, dtype, max_len=96)
            got = run_part(h, h.model.layers[layer].feed_forward, x, dtype, sizes)
            assert part_err(got, want) < PART_TOL[dtype], (name, layer, sizes)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["A", "B", "C", "D", "E"])
def test_stream_after_every_layer(tmp_path, dtype, name):
    import socrates_b200.engine.context as C
    from socrates_b200.parts.hyper import settled_sum
    folder, cfg, w = make_folder(tmp_path, name)
    ids = tokens(cfg["vocab"], 45, 11)
    want = []
    plain.forward(cfg, w, ids, layers_out=want)
    h = Harness(folder, dtype)
    got, ctxs = [], []

    original = C.StepContext.__init__

    def patched(self, *a, **k):
        original(self, *a, **k)
        self.after_run = lambda i, stream: got.append(settled_sum(self, stream).double().cpu())
    C.StepContext.__init__ = patched
    try:
        h.step([("a", ids)])
    finally:
        C.StepContext.__init__ = original
    assert len(got) == len(want) == len(cfg["layers"])
    for i, (a, b) in enumerate(zip(got, want)):
        assert part_err(a, b) < (1e-4 if dtype == torch.float32 else 5e-2), i


# ------------------------------------------------------------------------------------------
# whole models

@pytest.fixture(scope="module")
def models(tmp_path_factory):
    tmp = tmp_path_factory.mktemp("magedra")
    out = {}
    for name in TINY:
        folder, cfg, w = make_folder(tmp, name)
        seqs = [tokens(cfg["vocab"], n, 50 + i) for i, n in enumerate((150, 23, 77, 4))]
        out[name] = (folder, cfg, w, seqs, [plain.forward(cfg, w, s) for s in seqs])
    return out


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["A", "B", "C", "D", "E"])
def test_whole_prompts_decoding_and_portions(models, dtype, name):
    folder, cfg, w, seqs, want = models[name]
    h = Harness(folder, dtype)
    ids, ref = seqs[0], want[0]
    ways = {"whole": h.run("w", ids, (len(ids),)),
            "token by token": h.run("d", ids, (1,)),
            "pairs": h.run("p", ids, (2,)),
            "ragged": h.run("r", ids, (7, 2, 16, 3, 2, 33, 5, 17, 2, 1, 1, 1, 40)),
            "prompt then decoded": h.run("t", ids, (len(ids) - 100, 1))}
    for way, got in ways.items():
        assert rel_err(got, ref) < TOL[dtype], way
    if dtype == torch.float32:          # how the tokens were cut changes rounding only
        for way, got in ways.items():
            assert rel_err(got, ways["whole"]) < 2e-5, way
    # the first tokens of a sequence, alone
    assert rel_err(h.run("f", seqs[3], (1,)), want[3]) < TOL[dtype]
    assert rel_err(h.run("g", seqs[3], (4,)), want[3]) < TOL[dtype]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["A", "B", "C", "D", "E"])
def test_unequal_requests_in_one_batch(models, dtype, name):
    """Four requests of 150, 23, 77 and 4 tokens: portions of some beside single tokens of others, a
    request that joins late and one that sits steps out; each must come out as it does alone."""
    folder, cfg, w, seqs, want = models[name]
    h = Harness(folder, dtype)
    alone = [Harness(folder, dtype).run("x", s, (len(s),)) for s in seqs] if dtype == torch.float32 else None
    fed = [0] * 4
    got = [[] for _ in seqs]
    plan = [[(0, 60), (1, 1)], [(0, 1), (1, 1), (2, 30)], [(0, 2), (2, 1), (3, 4)], [(1, 20), (2, 1)],
            [(0, 30), (1, 1), (2, 44)], [(0, 1), (2, 1)], [(0, 56)]]
    for step in plan:
        entries = [(f"r{i}", seqs[i][fed[i]:fed[i] + c]) for i, c in step if fed[i] < len(seqs[i])]
        ended = [f"r{i}" for i, c in step if fed[i] < len(seqs[i]) and fed[i] + c >= len(seqs[i])]
        out = h.step(entries, end=ended)
        for i, c in step:
            if f"r{i}" in out:
                got[i].append(out[f"r{i}"])
                fed[i] += out[f"r{i}"].shape[0]
    for i, s in enumerate(seqs):
        mine = torch.cat(got[i])
        assert mine.shape[0] == len(s)
        assert rel_err(mine, want[i]) < TOL[dtype], i
        if alone is not None:
            assert rel_err(mine, alone[i]) < 2e-5, i


@pytest.mark.parametrize("dtype", DTYPES)
def test_rows_pages_and_state_slots_are_used_again(models, dtype):
    """Two rows and a pool of 12 pages of 16 slots serve eight requests one after another, in portions and token
    by token: every page is handed out several times, dirty from its previous owner, and every state slot
    starts from zero again although its last owner left a state behind."""
    folder, cfg, w, seqs, want = models["A"]
    h = Harness(folder, dtype, max_rows=2, max_len=160, pages=12)
    order = [0, 1, 2, 3, 2, 0, 3, 1]
    for k in range(0, len(order), 2):
        a, b = order[k], order[k + 1]
        ga = h.run(f"a{k}", seqs[a], (31, 1, 2, 64))
        fed, gb = 0, []
        while fed < len(seqs[b]):                       # the second of the pair decodes token by token
            gb.append(h.step([(f"b{k}", seqs[b][fed:fed + 1])], end=[f"b{k}"] if fed + 1 == len(seqs[b]) else [])[f"b{k}"])
            fed += 1
        assert rel_err(ga, want[a]) < TOL[dtype] and rel_err(torch.cat(gb), want[b]) < TOL[dtype], k
    assert h.cache.free_pages() == [12] * len(h.cache.groups) and len(h.cache.groups) == 2


PLANT = {"architecture": "Magedra", "vocab": 50, "width": 48, "norm": {"eps": 1e-6}, "residual_mult": 1.0, "streams": 2,
         "layers": [{"type": "parallel", "mlp": None,
                     "mixer": {"left": {"heads": 4, "kv_heads": 2, "dim": 8, "vdim": 24, "scale": 0.4},
                               "right": {"heads": 1, "dim": 4, "vdim": 4}, "left_scale": 1.0, "right_scale": 0.0}},
                    {"type": "latent_attention", "mlp": None,
                     "mixer": {"heads": 2, "dim": 8, "rot_dim": 0, "vdim": 12, "q_rank": 16, "kv_rank": 24, "scale": 0.4,
                               "rot": {"base": 100.0, "dims": 0}}}]}


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("layer", [0, 1])
def test_one_planted_key_decides_attention(tmp_path, dtype, layer):
    """A mixer alone, without rotation, so that a planted pair scores high at every distance: for the last
    queries the key at position `at` has by far the largest score, so its value is most of what they read.
    `at` is put far back among hundreds of keys, on the last and first slot of a page, on either side of a chunk
    of 128 keys of the last query, and right behind a query.  The planted key is read in a prompt, decoded, and
    from an earlier portion.  Layer 0: attention with mixed scores; layer 1: latent attention."""
    folder, cfg, w = make_folder(tmp_path, "plant", cfg=PLANT)
    spec = cfg["layers"][layer]
    eps, pre = cfg["norm"]["eps"], f"l{layer}.mix."
    n, width = 300, cfg["width"]
    last = n - 1
    places = {"far": 2, "end of a page": 15, "start of a page": 16, "before the last chunk": last - 128,
              "in the last chunk": last - 127, "start of the second chunk": 128, "near": last - 3}
    g = torch.Generator().manual_seed(8 + layer)
    for where, at in places.items():
        x = torch.randn(n, width, generator=g) * 1.5
        u = x[at] / x[at].norm()
        planted = x[at].clone()
        x = x - (x @ u)[:, None] * u[None, :]           # no other input has a component along the planted key's
        x[at] = planted
        x = x.bfloat16().double()
        for p in (last - 28, last - 12):                # the same query three times: in the prompt and decoded
            x[p] = x[last]
        w2 = dict(w)
        if layer == 0:
            wk, wq = w2[pre + "left.k"].clone(), w2[pre + "left.q"].clone()
            wk += 5.0 * x[at] / x[at].norm()
            wq += 5.0 * x[last] / x[last].norm()
            w2[pre + "left.k"], w2[pre + "left.q"] = wk.bfloat16().double(), wq.bfloat16().double()
        else:
            # both latents are normed, so a large input makes no large score: the up-projections get a rank-one
            # term along the planted token's latent (keys) and the last query's latent (queries) instead
            m = spec["mixer"]
            H, dn, rank = m["heads"], m["dim"], m["kv_rank"]
            c_at = plain.rms_norm(x[at] @ w[pre + "dkv"][:rank].T, w[pre + "dkv.norm"], eps)
            cq_last = plain.rms_norm(x[last] @ w[pre + "dq"].T, w[pre + "dq.norm"], eps)
            e = torch.ones(dn, dtype=F64) / dn ** 0.5
            uk = w2[pre + "uk"].clone().view(H, dn, rank) + 1.8 * e[None, :, None] * (c_at / c_at.norm())[None, None, :]
            uq = w2[pre + "uq"].clone().view(H, dn, -1) + 1.8 * e[None, :, None] * (cq_last / cq_last.norm())[None, None, :]
            w2[pre + "uk"], w2[pre + "uq"] = uk.reshape(H * dn, rank).bfloat16().double(), uq.reshape(H * dn, -1).bfloat16().double()
        save_weights(folder, w2)
        want = plain_mixer(spec["type"], x, w2, pre, spec["mixer"], eps)
        lost = x.clone()
        lost[at] = x[at + 1]
        gone = plain_mixer(spec["type"], lost, w2, pre, spec["mixer"], eps)
        assert part_err(gone[last:], want[last:]) > 0.2, where              # the planted key matters
        for sizes in ((n,), (last - 20, 1), (at + 1, 2, max(1, last - 20 - at - 3), 1)):
            h = Harness(folder, dtype, max_len=320)
            got = run_part(h, h.model.layers[layer].mixer, x, dtype, sizes, entry=layer)
            if dtype == torch.float32:
                assert part_err(got, want) < PART_TOL[dtype], (where, at, sizes)
                continue
            err = (got - want).abs().max(-1).values / want.abs().max()
            assert float(err[[last - 28, last - 12, last]].max()) < 0.08, (where, at, sizes)
            assert float(err.median()) < 0.02 and float(err.max()) < 0.15, (where, at, sizes)


@pytest.mark.parametrize("dtype", DTYPES)
def test_a_state_carries_one_write_over_hundreds_of_tokens(tmp_path, dtype):
    """Linear attention whose forget gate is one everywhere except at token 3: what token 3 writes is ALL that
    token 299 reads, in a prompt, decoded, and across portions (a lost or re-zeroed state reads nothing); the
    minGRU likewise with an update gate that is open at token 3 only."""
    cfg = json.loads(json.dumps(PLANT))
    cfg["layers"] = [{"type": "parallel", "mlp": None,
                      "mixer": {"left": {"heads": 1, "kv_heads": 1, "dim": 8, "vdim": 8, "scale": 0.1},
                                "right": {"heads": 2, "dim": 6, "vdim": 10}, "left_scale": 0.0, "right_scale": 1.0}},
                     {"type": "mingru", "mlp": None, "mixer": {"width": 20}}]
    folder, cfg, w = make_folder(tmp_path, "carry", cfg=cfg)
    n, width, eps = 300, cfg["width"], cfg["norm"]["eps"]
    g = torch.Generator().manual_seed(12)
    x = (torch.randn(n, width, generator=g)).bfloat16().double()
    u = x[3] / x[3].norm()
    planted = x[3].clone()
    x = x - (x @ u)[:, None] * u[None, :]               # no other input has a component along token 3's
    x[3] = planted
    x = x.bfloat16().double()
    w2 = dict(w)
    # linear attention: the forget gate is one (nothing is written, nothing forgotten) except at token 3, where
    # it falls to its lower bound of one half
    w2["l0.mix.right.lower"] = torch.full_like(w["l0.mix.right.lower"], 0.5)
    w2["l0.mix.right.f.b"] = torch.full_like(w["l0.mix.right.f.b"], 30.0)
    w2["l0.mix.right.f"] = (w["l0.mix.right.f"] - (60.0 / float(x[3].norm())) * u[None, :]).bfloat16().double()
    # minGRU: the update gate is shut except at token 3, where it is open
    w2["l1.mix.z.b"] = torch.full_like(w["l1.mix.z.b"], -30.0)
    w2["l1.mix.z"] = (w["l1.mix.z"] + (60.0 / float(x[3].norm())) * u[None, :]).bfloat16().double()
    save_weights(folder, w2)
    for layer, kind in ((0, "parallel"), (1, "mingru")):
        pre, m = f"l{layer}.mix.", cfg["layers"][layer]["mixer"]
        want = plain_mixer(kind, x, w2, pre, m, eps)
        lost = x.clone()
        lost[3] = x[4]
        gone = plain_mixer(kind, lost, w2, pre, m, eps)
        assert part_err(gone[-5:], want[-5:]) > 0.5, kind                    # token 3 is all that the end reads
        for sizes in ((n,), (280, 1), (4, 2, 150, 1)):
            h = Harness(folder, dtype, max_len=320)
            got = run_part(h, h.model.layers[layer].mixer, x, dtype, sizes, entry=layer)
            if dtype == torch.float32 or kind == "mingru":
                assert part_err(got, want) < PART_TOL[dtype], (kind, sizes)
                continue
            # every later token reads the one write through sum_d q_d, and the head norm leaves only the sign of
            # that sum: where bfloat16 rounds a sum near zero to the other side the row flips, so the rows are
            # judged one by one and a few may differ
            err = (got - want).abs().max(-1).values / want.abs().max()
            assert float(err.quantile(0.9)) < PART_TOL[dtype] and float(err.median()) < 0.01, (kind, sizes)


def test_long_decoding(models):
    """400 tokens decoded one by one after a short prompt, two requests side by side, in float32."""
    for name in ("B", "D"):
        folder, cfg, w, _, _ = models[name]
        a, b = tokens(cfg["vocab"], 410, 77), tokens(cfg["vocab"], 300, 78)
        ra, rb = plain.forward(cfg, w, a), plain.forward(cfg, w, b)
        h = Harness(folder, torch.float32, max_len=448)
        ga, gb = [h.step([("a", a[:10])])["a"]], []
        for t in range(10, 410):
            entries = [("a", a[t:t + 1])]
            if t - 10 < 300:
                entries.append(("b", b[t - 10:t - 9]))
            out = h.step(entries)
            ga.append(out["a"])
            if "b" in out:
                gb.append(out["b"])
        assert rel_err(torch.cat(ga), ra) < TOL[torch.float32] and rel_err(torch.cat(gb), rb) < TOL[torch.float32]


# ------------------------------------------------------------------------------------------
# the entry point, the scheduler, the command-line replay

@pytest.mark.parametrize("dtype,graphs", [("float32", False), ("bfloat16", True)])
@pytest.mark.parametrize("name", ["A", "B", "C", "E"])
def test_greedy_generation_through_the_entry_point(models, name, dtype, graphs):
    """Five requests through Engine: queued, admitted as rows come free, prompts cut by the token
    budget, decoded side by side (bfloat16: through recorded graphs), 90 new tokens each.  Every
    produced token is the plain statement's choice, or within its margin."""
    from socrates_b200 import Engine
    folder, cfg, w, seqs, _ = models[name]
    prompts = [seqs[0][:70], seqs[1], seqs[2][:40], seqs[3], seqs[0][70:101]]
    eng = Engine(str(folder), device="cuda:0", dtype=dtype, compile=graphs, max_batch=3, max_len=192,
                 max_new_tokens=90, token_budget=48)
    reqs = [eng.submit(p) for p in prompts]
    while eng.scheduler.has_work():
        assert eng.step()
        eng.scheduler.check()
    margin = 1e-3 if dtype == "float32" else 8e-2
    for p, r in zip(prompts, reqs):
        assert r.done and len(r.output) == 90
        logits = plain.forward(cfg, w, list(p) + r.output[:-1])
        scale = float(logits.abs().max())
        for i, tok in enumerate(r.output):
            row = logits[len(p) - 1 + i]
            best = int(torch.argmax(row))
            assert tok == best or float(row[best] - row[tok]) <= margin * scale, (i, tok, best)
    eng.cache.check()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_replay_program(models, tmp_path, dtype):
    """bin/trace_run on model A: whole, tail decoded, portions, and a mix of up to four live requests
    in a pool that only holds the busiest step."""
    folder, cfg, w, seqs, want = models["A"]
    named = {f"s{i}": s for i, s in enumerate(seqs[:3])}
    reference = {k: want[i].numpy() for i, k in enumerate(named)}
    trace = Trace()
    for k, ids in named.items():
        whole(trace, "w:" + k, ids)
        last_decoded(trace, "d:" + k, ids, tail=20)
        portions(trace, "p:" + k, ids)
    mixed(trace, {f"m{j}:{k}": ids for j in range(2) for k, ids in named.items()}, seed=5, tail=20)
    result = run_trace(folder, dtype, trace, trace.most_held, tmp_path / "out")
    worst, where = compare(trace, result, reference, key=lambda rid: rid.split(":")[1])
    assert worst < TOL[torch.float32 if dtype == "float32" else torch.bfloat16], where


def test_command_line(models, tmp_path):
    """The generation command line on a Magedra folder, and on a bare config.json with random weights."""
    import subprocess
    import sys
    from pathlib import Path
    root = Path(__file__).resolve().parent.parent
    folder, cfg, _, _, _ = models["A"]
    common = ["--max-new-tokens", "7", "--max-len", "96", "--max-batch", "2"]
    proc = subprocess.run([sys.executable, "-m", "socrates_b200.inference_paged", "--model", str(folder),
                           "--num-prompts", "3", "--prompt-len", "21", "--prompt", "hello", *common],
                          cwd=str(root), capture_output=True, text=True, timeout=300)
    assert proc.returncode == 0, proc.stderr[-2000:]
    assert "4 requests, 2 rows" in proc.stdout and "> hello" in proc.stdout
    path = tmp_path / "config.json"
    path.write_text(json.dumps(TINY["B"]))
    proc = subprocess.run([sys.executable, "-m", "socrates_b200.inference_paged", "--random-config", str(path),
                           "--num-prompts", "2", "--prompt-len", "30", "--dtype", "float32", *common],
                          cwd=str(root), capture_output=True, text=True, timeout=300)
    assert proc.returncode == 0, proc.stderr[-2000:]
    assert "2 requests, 2 rows" in proc.stdout and "tok/s" in proc.stdout.splitlines()[-1]
