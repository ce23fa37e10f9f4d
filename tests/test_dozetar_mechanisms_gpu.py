"""Dozetar's mechanisms one at a time on the GPU kernels, each against its plain restatement: the
output-normed residual add, the logit cap, the gated group norm, the two matrix-state recurrences
(steps, slots, odd sizes), the sink attention (windows, kept first tokens, pages, far keys) and the
sigmoid-scored experts whose weight scales their input."""
import pytest
import torch

import dozetar_plain as P
import dozetar_util as U

pytestmark = pytest.mark.gpu
DEV = "cuda"
TOL = {torch.float32: 2e-5, torch.bfloat16: 2e-2}


def _err(got, want):
    return float((got.double().cpu() - want).abs().max() / want.abs().max().clamp_min(1e-9))


# ---- residual add with the norm on the sublayer's output ---------------------------------------------
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("width", [40, 333])
def test_add_normed_terms_and_copy(dtype, width):
    from sglang_security_b200.layers.residual_norm import AddNormed

    g = torch.Generator().manual_seed(1)
    T, top = 7, 3
    x = torch.randn(T, width, generator=g)
    a, b = (torch.randn(T, width, generator=g).to(dtype) for _ in range(2))
    rows = torch.randn(T * top, width, generator=g).to(dtype)
    mod = AddNormed(width, 1e-3, mult=0.25).to(DEV)
    mod.weight.data.copy_(1 + 0.3 * torch.randn(width, generator=g))
    w = mod.weight.double().cpu()
    for kw, y in (({"a": a}, a.double()), ({"a": a, "sa": 0.6, "b": b, "sb": -1.1}, 0.6 * a.double() - 1.1 * b.double()),
                  ({"rows": rows, "top": top}, rows.double().view(T, top, width).sum(1))):
        xs = x.clone().to(DEV)
        h = mod(xs, out_dtype=dtype, **{k: (v.to(DEV) if torch.is_tensor(v) else v) for k, v in kw.items()})
        want = x.double() + 0.25 * P.rms(y, 1e-3) * w
        assert _err(xs, want) <= 2e-6
        assert torch.equal(h.float().cpu(), xs.cpu().to(dtype).float())


def test_softcap_rows():
    from sglang_security_b200.layers.residual_norm import softcap

    z = torch.linspace(-90, 90, 600).view(3, -1)
    assert _err(softcap(z.to(DEV), 25.0), 25.0 * torch.tanh(z.double() / 25.0)) <= 1e-6
    assert torch.equal(softcap(z.to(DEV).bfloat16(), 0.0).cpu(), z.bfloat16().float())


def test_gated_group_rmsnorm_divides_by_the_recurrence_normaliser():
    from sglang_security_b200.layers.recurrent.linear_recurrence import gated_group_rmsnorm

    g = torch.Generator().manual_seed(3)
    T, H, E = 6, 3, 10
    o, w = torch.randn(T, H * E, generator=g), 1 + 0.3 * torch.randn(H * E, generator=g)
    aux = torch.cat([torch.randn(T, H, generator=g) * 3, torch.randn(T, H, generator=g)], 1)
    got = gated_group_rmsnorm(o.to(DEV), w.to(DEV), None, E, 1e-4, torch.float32, aux=aux.to(DEV), heads=H, den_eps=1e-6)
    den = torch.maximum(aux[:, :H].abs(), torch.exp(-aux[:, H:])).double() + 1e-6
    y = P.rms(o.double().view(T, H, E) / den[:, :, None], 1e-4).reshape(T, H * E) * w.double()
    assert _err(got, y) <= 1e-5


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("heads,vdim,whole", [(3, 20, False), (3, 20, True), (1, 7, False), (9, 64, True)])
def test_gated_group_rmsnorm(dtype, heads, vdim, whole):
    from sglang_security_b200.layers.recurrent.linear_recurrence import gated_group_rmsnorm

    g = torch.Generator().manual_seed(2)
    T, N = 11, heads * vdim
    o = torch.randn(T, N, generator=g) * 3
    w = 1 + 0.3 * torch.randn(N, generator=g)
    z = torch.randn(T, N, generator=g).to(dtype)
    got = gated_group_rmsnorm(o.to(DEV), w.to(DEV), z.to(DEV), N if whole else vdim, 1e-4, dtype)
    y = P.rms(o.double(), 1e-4) if whole else P.rms(o.double().view(T, heads, vdim), 1e-4).reshape(T, N)
    assert _err(got, y * w.double() * torch.sigmoid(z.double())) <= (1e-5 if dtype == torch.float32 else 8e-3)


# ---- recurrences ---------------------------------------------------------------------------------------
def _run_recurrence(gated, H, D, E, lens, cuts, dtype, seed=0, cap=6.0, reuse=False):
    """`lens` sequences fed together in portions `cuts[i]`; -> (outputs per sequence, oracle per sequence)."""
    from sglang_security_b200.layers.recurrent.linear_recurrence import linear_recurrence, state_width

    g = torch.Generator().manual_seed(seed)
    hb = U.HandBatch(len(lens), max(lens) + 1)
    state = torch.full((len(lens), state_width(H, D, E, gated)), 7.0, device=DEV)      # stale values everywhere
    decay = torch.tensor([0.3 + 0.69 * i / max(1, H - 1) for i in range(H)])
    data = []
    for n in lens:
        q, k = (torch.randn(n, H * D, generator=g).to(dtype) for _ in range(2))
        v = torch.randn(n, H * E, generator=g).to(dtype)
        gates = torch.randn(n, 2 * H, generator=g) * 3 + torch.tensor([0.0] * H + [2.0] * H)
        data.append((q, k, v, gates))
    got = [[] for _ in lens]
    at = [0] * len(lens)
    todo = [list(c) for c in cuts]
    while any(todo):
        entries = [(i, todo[i].pop(0)) for i in range(len(lens)) if todo[i]]
        fb = hb.step(entries)
        part = [torch.cat([data[i][j][at[i]:at[i] + n] for i, n in entries]).to(DEV) for j in range(4)]
        out = linear_recurrence(part[0], part[1], part[2], H, D, E, state, fb,
                                gates=part[3] if gated else None, decay=None if gated else decay.to(DEV),
                                cap=cap, q_scale=D ** -0.5 if gated else 1.0, silu=not gated)
        if gated:          # (un-normalised o, (n . q, m)): the division the norm kernel fuses, done here
            num, aux = out
            den = torch.maximum(aux[:, :H].abs(), torch.exp(-aux[:, H:])) + 1e-6
            out = (num.view(-1, H, E) / den[:, :, None]).view(-1, H * E)
        o = 0
        for i, n in entries:
            got[i].append(out[o:o + n].cpu())
            at[i] += n
            o += n
    want = []
    for (q, k, v, gates), n in zip(data, lens):
        qd, kd, vd = q.double().view(n, H, D), k.double().view(n, H, D), v.double().view(n, H, E)
        if gated:
            li = P.capped(gates[:, :H].double(), cap)
            lf = torch.nn.functional.logsigmoid(P.capped(gates[:, H:].double(), cap))
            want.append(P.mlstm_recurrence(qd * D ** -0.5, kd, vd, li, lf).reshape(n, H * E))
        else:
            s = torch.nn.functional.silu
            want.append(P.decayed_recurrence(s(qd), s(kd), s(vd), decay.tolist()).reshape(n, H * E))
    return [torch.cat(x) for x in got], want


@pytest.mark.parametrize("gated", [False, True])
@pytest.mark.parametrize("H,D,E", [(2, 16, 16), (3, 24, 20), (1, 40, 72), (2, 72, 9), (4, 1, 1), (1, 130, 33)])
def test_recurrence_portions_against_token_by_token(gated, H, D, E):
    lens = [37, 5, 61]
    cuts = [U.cut(37, [2, 5, 1, 16]), [5], U.cut(61, [33, 1, 1, 2])]
    got, want = _run_recurrence(gated, H, D, E, lens, cuts, torch.float32)
    for a, b in zip(got, want):
        assert _err(a, b) <= 5e-5
    one, _ = _run_recurrence(gated, H, D, E, lens, [[1] * n for n in lens], torch.float32)
    for a, b in zip(got, one):
        assert torch.equal(a, b)        # the same sums in the same order however the sequence is cut


@pytest.mark.parametrize("gated", [False, True])
def test_recurrence_bf16_inputs_and_long_decode(gated):
    got, want = _run_recurrence(gated, 2, 32, 48, [420], [[20] + [1] * 400], torch.bfloat16, seed=5)
    assert _err(got[0], want[0]) <= 1e-4


@pytest.mark.parametrize("gated", [False, True])
def test_recurrence_cta_sizes_share_one_state_layout(gated):
    """A few long portions split a head's columns over several CTAs, a wide batch of decoded tokens gives
    each head one large CTA: the state one launch leaves must be the state the other reads."""
    from sglang_security_b200 import _lib

    H, D, E, B = 8, 64, 128, 24
    cuts = [[12] + [1] * 3 for _ in range(B)]
    got, want = _run_recurrence(gated, H, D, E, [15] * B, cuts, torch.float32, seed=9)
    wide = _lib.last_variant()                      # the last step: 24 single tokens side by side
    for a, b in zip(got, want):
        assert _err(a, b) <= 5e-5
    one, _ = _run_recurrence(gated, H, D, E, [15], [[12, 1, 1, 1]], torch.float32, seed=9)
    assert _lib.last_variant() != wide
    assert _err(one[0], want[0]) <= 5e-5


def test_recurrence_state_of_a_reused_slot_is_ignored():
    from sglang_security_b200.layers.recurrent.linear_recurrence import linear_recurrence, state_width

    H, D, E = 2, 8, 8
    g = torch.Generator().manual_seed(6)
    hb = U.HandBatch(1, 64)
    state = torch.zeros((1, state_width(H, D, E, True)), device=DEV)
    outs = []
    for rep in range(2):
        q, k, v = (torch.randn(9, H * D, generator=torch.Generator().manual_seed(7)).to(DEV) for _ in range(3))
        gates = torch.randn(9, 2 * H, generator=torch.Generator().manual_seed(8)).to(DEV)
        fb = hb.step([(0, 9)])
        outs.append(torch.cat(linear_recurrence(q, k, v, H, D, E, state, fb, gates=gates, cap=0.0), 1))
        hb.release(0)                     # the next sequence in this row starts at position 0
    assert torch.equal(outs[0], outs[1]) and state.abs().max() > 0


# ---- attention with window, kept first tokens and sink -----------------------------------------------
def _attend(q, k, v, sink, scale, window, keep_first, cuts, dtype, page=16, seed=0, tensor_core=False):
    """One sequence through qk_norm_rope_write (norm and rotation off) + sink_attn in portions `cuts`;
    tensor_core: the portions run on the tcgen05 extend kernel instead of the CUDA-core one."""
    from sglang_security_b200 import _lib

    T, H, D = q.shape
    G, E = k.shape[1], v.shape[2]
    hb = U.HandBatch(2, T + page, page=page, seed=seed)
    hb.step([(1, 3)])                                   # another request owns the first pages handed out
    pool = torch.full((hb.pool_rows, G * (D + E)), 3.0, dtype=dtype, device=DEV)
    lib, code = _lib.load(), _lib.dtype_code(dtype)
    outs, at = [], 0
    for n in cuts:
        fb = hb.step([(0, n)])
        qq, kk, vv = (t[at:at + n].reshape(n, -1).to(dtype).to(DEV).contiguous() for t in (q, k, v))
        q32 = torch.empty((n, H * D), dtype=torch.float32, device=DEV)
        q16 = torch.empty((n, H * D), dtype=dtype, device=DEV)
        rc = lib.b200_qk_norm_rope_write(qq.data_ptr(), qq.stride(0), kk.data_ptr(), kk.stride(0), vv.data_ptr(),
                                         vv.stride(0), None, None, 0, 0, 1e-6, None, None, 0, fb.tok_pos.data_ptr(),
                                         fb.out_cache_loc.data_ptr(), pool.data_ptr(), pool.stride(0), 0, G * D,
                                         q32.data_ptr(), q32.stride(0), q16.data_ptr(), q16.stride(0), n, H, G, D, E,
                                         code, 0)
        _lib.check(rc, "prep")
        out = torch.empty((n, H * E), dtype=dtype, device=DEV)
        sink_d = sink.float().to(DEV) if sink is not None else None
        if tensor_core:
            i32 = lambda x: torch.tensor([x], dtype=torch.int32, device=DEV)
            seq, pre, ext, start = torch.tensor([at + n], device=DEV), i32(at), i32(n), i32(0)
            rc = lib.b200_attn_extend_sink(
                q16.data_ptr(), q16.stride(0), pool.data_ptr(), pool[:, G * D:].data_ptr(), pool.stride(0),
                out.data_ptr(), out.stride(0), fb.req_to_token.data_ptr(), fb.req_to_token.stride(0),
                fb.req_pool_indices.data_ptr(), seq.data_ptr(), pre.data_ptr(), ext.data_ptr(), start.data_ptr(), 1, n,
                H, G, D, E, scale, 0.0, 1.0, 1, window or 0, keep_first, _lib.ptr(sink_d), code, 0)
            _lib.check(rc, "extend")
            torch.cuda.synchronize()
            outs.append(out.cpu())
            at += n
            continue
        rc = lib.b200_sink_attn(q32.data_ptr(), q32.stride(0), pool.data_ptr(), pool.stride(0), 0, G * D,
                                fb.req_to_token.data_ptr(), fb.req_to_token.stride(0), fb.req_pool_indices.data_ptr(),
                                fb.tok_pos.data_ptr(), fb.tok_b.data_ptr(), _lib.ptr(sink_d),
                                scale, window or 0, keep_first, out.data_ptr(), out.stride(0), n, H, G, D, E, None, at + n if seed % 2 == 0 else 0, code, 0)
        _lib.check(rc, "attn")
        torch.cuda.synchronize()
        outs.append(out.cpu())
        at += n
    return torch.cat(outs).view(T, H, E)


def _qkv(T, H, G, D, E, seed, dtype):
    g = torch.Generator().manual_seed(seed)
    r = lambda *s: torch.randn(*s, generator=g).to(dtype).double()
    return r(T, H, D), r(T, G, D), r(T, G, E)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,G,D,E,window,keep", [(4, 2, 16, 24, 9, 2), (6, 2, 48, 80, 40, 5), (2, 2, 8, 8, 1, 0),
                                                 (3, 1, 10, 5, None, 0), (1, 1, 24, 130, 33, 35), (2, 1, 6, 3, 5, 1),
                                                 (10, 1, 12, 20, 17, 3), (16, 2, 8, 8, 64, 0)])
def test_sink_attention_prefill_portions_decode(dtype, H, G, D, E, window, keep):
    T = 150
    q, k, v = _qkv(T, H, G, D, E, 11, dtype)
    sink = torch.randn(H, generator=torch.Generator().manual_seed(12))
    want = P.sink_softmax(q, k, v, D ** -0.5, window, keep, sink.double())
    for cuts in ([T], U.cut(T, [2, 31, 1, 1, 17]), [100] + [1] * 50):
        got = _attend(q, k, v, sink, D ** -0.5, window, keep, cuts, dtype)
        assert _err(got, want) <= TOL[dtype], cuts[:3]


@pytest.mark.parametrize("decode", [False, True])
def test_window_edges_kept_tokens_and_far_keys_stand_out(decode):
    """One key gets a score far above the rest and a value no other key has: whether it is seen decides
    the output.  The key sits just inside / just outside the window, among the kept first tokens / right
    after them, on a page border, and hundreds of tokens back."""
    T, H, G, D, E, window, keep = 400, 2, 1, 16, 8, 37, 3
    base_q, base_k, base_v = _qkv(T, H, G, D, E, 21, torch.float32)
    sink = torch.zeros(H)
    query = T - 1
    cases = {query - window + 1: True, query - window: False, keep - 1: True, keep: False, 0: True,
             query - 16: True, 15: False, query: True}
    for key, seen in cases.items():
        q, k, v = base_q.clone(), base_k.clone() * 0.1, base_v.clone()
        k[key, 0] = q[query, 0] / q[query, 0].norm() * 40.0
        v[key, 0] = 100.0
        cuts = [T - 5] + [1] * 5 if decode else [T]
        got = _attend(q, k, v, sink, 1.0, window, keep, cuts, torch.float32)[query, 0]
        want = P.sink_softmax(q, k, v, 1.0, window, keep, sink.double())[query, 0]
        assert _err(got, want) <= 1e-4
        assert (got.abs().max() > 50) == seen, (key, seen)
    # without a window the farthest key is seen
    q, k, v = base_q.clone(), base_k.clone() * 0.1, base_v.clone()
    k[1, 0] = q[query, 0] / q[query, 0].norm() * 40.0
    v[1, 0] = 100.0
    got = _attend(q, k, v, sink, 1.0, None, 0, [T - 1, 1] if decode else [T], torch.float32)[query, 0]
    assert got.abs().max() > 50


@pytest.mark.parametrize("H,G,D,window,keep", [(4, 2, 64, 40, 4), (8, 1, 128, 200, 70), (2, 2, 64, 7, 0),
                                               (6, 2, 128, None, 0), (3, 3, 64, 130, 129), (16, 2, 64, 65, 1)])
def test_sink_attention_on_the_tensor_core_kernel(H, G, D, window, keep):
    T = 450
    q, k, v = _qkv(T, H, G, D, D, 61, torch.bfloat16)
    sink = torch.randn(H, generator=torch.Generator().manual_seed(62)) + 1.0
    want = P.sink_softmax(q, k, v, D ** -0.5, window, keep, sink.double())
    for cuts in ([T], [200, 130, 1, 119], [63, 64, 65, 258]):
        got = _attend(q, k, v, sink, D ** -0.5, window, keep, cuts, torch.bfloat16, tensor_core=True)
        assert _err(got, want) <= TOL[torch.bfloat16], cuts


def test_tensor_core_kernel_sees_the_edges():
    """As above with one outstanding key: just inside / outside the window, among / after the kept
    tokens, at tile borders (64 keys), far back."""
    T, H, G, D, window, keep = 400, 2, 1, 64, 100, 3
    base_q, base_k, base_v = _qkv(T, H, G, D, D, 63, torch.bfloat16)
    query = T - 1
    cases = {query - window + 1: True, query - window: False, keep - 1: True, keep: False, 0: True, 63: False,
             64: False, 320: True, 319: True, query: True}
    for key, seen in cases.items():
        q, k, v = base_q.clone(), base_k.clone() * 0.1, base_v.clone()
        k[key, 0] = (q[query, 0] / q[query, 0].norm() * 40.0).bfloat16().double()
        v[key, 0] = 100.0
        for cuts in ([T], [T - 70, 70]):
            got = _attend(q, k, v, torch.zeros(H), 1.0, window, keep, cuts, torch.bfloat16, tensor_core=True)[query, 0]
            assert (got.abs().max() > 50) == seen, (key, seen, cuts)
        want = P.sink_softmax(q, k, v, 1.0, window, keep, torch.zeros(H, dtype=P.DT))[query, 0]
        assert _err(got, want) <= 2e-2


def test_sink_changes_the_denominator_only():
    T, H, G, D, E = 20, 2, 2, 8, 8
    q, k, v = _qkv(T, H, G, D, E, 31, torch.float32)
    plain = _attend(q, k, v, None, 0.3, None, 0, [T], torch.float32)
    low = _attend(q, k, v, torch.full((H,), -80.0), 0.3, None, 0, [T], torch.float32)
    big = _attend(q, k, v, torch.tensor([5.0, -80.0]), 0.3, None, 0, [T], torch.float32)
    assert torch.allclose(plain, low, atol=1e-6)
    want = P.sink_softmax(q, k, v, 0.3, None, 0, torch.tensor([5.0, -80.0], dtype=P.DT))
    assert _err(big, want) <= 2e-5 and big[:, 0].abs().max() < plain[:, 0].abs().max()


@pytest.mark.parametrize("group", ["whole", "head"])
def test_qk_norm_and_partial_rotation(group):
    """Norm over the whole projection (or per head) with a weight, then interleaved pairs on the first
    rotated coordinates only, at positions far from 0."""
    from sglang_security_b200 import _lib

    H, G, D, E, dims, base, eps = 3, 1, 10, 4, 6, 250000.0, 1e-3
    g = torch.Generator().manual_seed(41)
    n, first = 5, 70000
    q, k, v = torch.randn(n, H * D, generator=g), torch.randn(n, G * D, generator=g), torch.randn(n, G * E, generator=g)
    qw, kw = 1 + 0.3 * torch.randn(H * D, generator=g), 1 + 0.3 * torch.randn(G * D, generator=g)
    pos = torch.arange(first, first + n, dtype=torch.int32)
    loc = torch.tensor([9, 3, 4, 0, 7], dtype=torch.int64)
    pool = torch.zeros((12, G * (D + E)), device=DEV)
    f = torch.tensor([base ** (-2.0 * i / dims) for i in range(dims // 2)], dtype=torch.float64)
    hi = f.float()
    lo = (f - hi.double()).float()
    q32 = torch.empty((n, H * D), device=DEV)
    qg, kg = (H * D, G * D) if group == "whole" else (D, D)
    qd, kd, vd, qwd, kwd, hid, lod, posd, locd = (t.to(DEV) for t in (q, k, v, qw, kw, hi, lo, pos, loc))
    rc = _lib.load().b200_qk_norm_rope_write(
        qd.data_ptr(), qd.stride(0), kd.data_ptr(), kd.stride(0), vd.data_ptr(), vd.stride(0), qwd.data_ptr(),
        kwd.data_ptr(), qg, kg, eps, hid.data_ptr(), lod.data_ptr(), dims, posd.data_ptr(),
        locd.data_ptr(), pool.data_ptr(), pool.stride(0), 0, G * D, q32.data_ptr(), q32.stride(0), None, 0, n, H, G,
        D, E, _lib.F32, 0)
    _lib.check(rc, "prep")

    def want(x, w, heads):
        y = x.double()
        y = P.rms(y, eps) if group == "whole" else P.rms(y.view(n, heads, D), eps).reshape(n, -1)
        return P.rotate_pairs((y * w.double()).view(n, heads, D), pos, dims, base).reshape(n, -1)

    assert _err(q32, want(q, qw, H)) <= 3e-6
    assert _err(pool[loc.to(DEV), :G * D], want(k, kw, G)) <= 3e-6
    assert torch.equal(pool[loc.to(DEV), G * D:].cpu(), v)


# ---- experts ---------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("E,top,ff,T", [(5, 2, 24, 3), (12, 1, 72, 150), (3, 3, 8, 1), (33, 4, 40, 70)])
def test_sigmoid_router_and_scaled_input_experts(dtype, E, top, ff, T):
    from sglang_security_b200.layers.moe.fused_moe import ScaledInputExperts, TopKRouter

    W = 40
    g = torch.Generator().manual_seed(51)
    x = torch.randn(T, W, generator=g)
    w = {"router": (torch.randn(E, W, generator=g) * 0.5).bfloat16()}
    for e in range(E):
        w[f"e{e}.up"] = (torch.randn(ff, W, generator=g) / W ** 0.5).bfloat16()
        w[f"e{e}.down"] = (torch.randn(W, ff, generator=g) / ff ** 0.5).bfloat16()
    router = TopKRouter(W, E, top, bias=False, score="sigmoid").to(DEV)
    router.weight.data.copy_(w["router"].float())
    ex = ScaledInputExperts(W, ff, E, "relu2", dtype).to(DEV)
    for e in range(E):
        ex.w_up.data[e].copy_(w[f"e{e}.up"])
        ex.w_down.data[e].copy_(w[f"e{e}.down"])
    h = x.to(dtype)
    ids, wts, _ = router(h.float().to(DEV))     # router and experts see the same values, as the oracle's do
    s = torch.sigmoid(h.double() @ w["router"].double().t())
    assert torch.equal(ids.cpu().long().sort(-1).values, torch.topk(s, top, -1).indices.sort(-1).values)
    assert _err(wts, torch.gather(s, 1, ids.cpu().long())) <= 1e-5
    rows = ex(h.to(DEV), ids, wts)
    got = rows.double().view(T, top, W).sum(1)
    want = P.moe(h.double(), w, "", {"router": {"experts": E, "top": top}})
    assert _err(got, want) <= (1e-5 if dtype == torch.float32 else 2e-2)
    # the weight is not a factor on the output: doubling it must quadruple a squared-relu expert
    rows2 = ex(h.to(DEV), ids, wts * 2)
    assert _err(rows2.double(), 4 * rows.double().cpu()) <= (1e-5 if dtype == torch.float32 else 2e-2)
