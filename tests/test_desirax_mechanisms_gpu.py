"""Each Desirax mechanism alone: the package's layer (CUDA kernels) against the plain restatement in
desirax_plain.py, on sizes that are not powers of two and not multiples of the kernels' tiles."""
from types import SimpleNamespace

import pytest
import torch

import desirax_plain as P

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _meta(chunks):
    """chunks: list of (start position, length) per batch entry -> the per-token tables."""
    pos, tb, start, ln, at = [], [], [], [], 0
    for b, (p0, n) in enumerate(chunks):
        pos += list(range(p0, p0 + n))
        tb += [b] * n
        start.append(at)
        ln.append(n)
        at += n
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=DEV)
    return SimpleNamespace(tok_pos=i32(pos), tok_b=i32(tb), ext_start=i32(start), ext_len=i32(ln))


@pytest.mark.parametrize("width", [40, 257, 1024])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_scalar_norm_and_token_shift_across_steps(width, dtype):
    from sglang_security_b200.layers.scalar_norm import ScalarRMSNorm, TokenShift

    torch.manual_seed(width)
    eps, gain = 1e-5, 1.3
    norm, shift = ScalarRMSNorm(eps).to(DEV), TokenShift(width).to(DEV)
    norm.gain.data.fill_(gain)
    shift.mu.data.copy_(torch.rand(width))
    seqs = [torch.randn(n, width) * 3 for n in (11, 1, 6)]
    want_h = [P.scalar_norm(s.double(), gain, eps) for s in seqs]
    want_hm = [P.token_shift(h, shift.mu.double().cpu()) for h in want_h]
    state = torch.full((5, width), 7.0, device=DEV)          # dirty slots: position 0 must not read them
    slots = torch.tensor([3, 0, 4], dtype=torch.int64, device=DEV)
    # three steps with unequal portions; sequence 1 (one token) is only in the first
    plan = [[(0, 0, 4), (1, 0, 1), (2, 0, 2)], [(0, 4, 1), (2, 2, 3)], [(0, 5, 6), (2, 5, 1)]]
    got_h = [[] for _ in seqs]
    got_hm = [[] for _ in seqs]
    for step in plan:
        x = torch.cat([seqs[s][p0:p0 + n] for s, p0, n in step]).to(DEV)
        meta = _meta([(p0, n) for _, p0, n in step])
        sl = slots[[s for s, _, _ in step]]
        h, hm = norm.forward_shifted(x, dtype, shift, meta, state, sl)
        at = 0
        for s, p0, n in step:
            got_h[s].append(h[at:at + n].double().cpu())
            got_hm[s].append(hm[at:at + n].double().cpu())
            at += n
    tol = 2e-6 if dtype == torch.float32 else 2e-2
    for s in range(3):
        assert (torch.cat(got_h[s]) - want_h[s]).abs().max() <= tol * want_h[s].abs().max()
        assert (torch.cat(got_hm[s]) - want_hm[s]).abs().max() <= tol * want_h[s].abs().max()
    # the carried row is the fp32 normed row of each sequence's last token
    assert (state[3].double().cpu() - want_h[0][-1]).abs().max() <= 2e-6 * want_h[0].abs().max()
    # plain norm (no shift) of arbitrary rows
    x = torch.randn(9, width, device=DEV)
    out = norm(x, dtype).double().cpu()
    assert (out - P.scalar_norm(x.double().cpu(), gain, eps)).abs().max() <= tol * 4


@pytest.mark.parametrize("act", ["silu", "gelu_tanh"])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_gated_feed_forward(act, dtype):
    from sglang_security_b200.layers.gated_mlp import GatedMLP

    torch.manual_seed(1)
    width, ff, n = 72, 100, 37
    g, u, d = (torch.randn(ff, width) / 8).bfloat16(), (torch.randn(ff, width) / 8).bfloat16(), \
        (torch.randn(width, ff) / 10).bfloat16()
    mlp = GatedMLP(width, ff, act, dtype).to(DEV)
    mlp.load(g.to(DEV).to(dtype), u.to(DEV).to(dtype), d.to(DEV).to(dtype))
    h = torch.randn(n, width).bfloat16()
    want = P.gated_ff(h.double(), g.double(), u.double(), d.double(), P.silu if act == "silu" else P.gelu_tanh)
    got = mlp(h.to(DEV).to(dtype)).double().cpu()
    assert (got - want).abs().max() <= (1e-5 if dtype == torch.float32 else 3e-2) * want.abs().max()


@pytest.mark.parametrize("experts,top", [(5, 2), (16, 1), (33, 4), (7, 7)])
def test_router_top_k_and_softmax_over_the_chosen(experts, top):
    from sglang_security_b200.layers.moe.fused_moe import TopKRouter

    torch.manual_seed(experts)
    width, n = 88, 53
    r = TopKRouter(width, experts, top, bias=True, shared_gate=True).to(DEV)
    r.weight.data.copy_(torch.randn(experts, width))
    r.bias.data.copy_(torch.randn(experts) * 2)      # a bias large enough to change the choice
    r.shared_gate.data.copy_(torch.randn(width) / 4)
    h = torch.randn(n, width)
    ids, wts, gate = r(h.to(DEV))
    wi, ww = P.route(h.double(), r.weight.double().cpu(), r.bias.double().cpu(), top)
    assert torch.equal(ids.cpu().long(), wi)
    assert (wts.cpu().double() - ww).abs().max() < 1e-5
    assert abs(float(wts.sum(-1).min()) - 1) < 1e-5
    want_gate = torch.sigmoid(h.double() @ r.shared_gate.double().cpu())
    assert (gate.cpu().double() - want_gate).abs().max() < 1e-5
    # without the bias the choice differs somewhere: the bias is really used
    assert not torch.equal(P.route(h.double(), r.weight.double().cpu(), torch.zeros(experts).double(), top)[0], wi)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_router_long_portion_matches_each_token_alone(dtype):
    """A long portion gives every token bit for bit what it gets when routed alone, and the plain
    router's choice."""
    from sglang_security_b200.layers.moe.fused_moe import TopKRouter

    torch.manual_seed(4)
    width, n, experts, top = 200, 1029, 12, 3
    r = TopKRouter(width, experts, top, bias=True, shared_gate=True).to(DEV)
    r.weight.data.copy_(torch.randn(experts, width))
    r.bias.data.copy_(torch.randn(experts))
    r.shared_gate.data.copy_(torch.randn(width) / 4)
    h = torch.randn(n, width).to(dtype)
    ids, wts, gate = r(h.to(DEV))
    wi, ww = P.route(h.double(), r.weight.double().cpu(), r.bias.double().cpu(), top)
    assert torch.equal(ids.cpu().long(), wi)
    assert (wts.cpu().double() - ww).abs().max() < 1e-5
    for t in (0, 7, 8, 1023, 1024, 1028):
        i1, w1, g1 = r(h[t:t + 1].to(DEV))
        assert torch.equal(i1[0], ids[t]) and torch.equal(w1[0], wts[t]) and torch.equal(g1[0], gate[t])


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("n", [1, 3, 150, 700])      # 700: the 16-bit kernel's 128-row tiles
def test_experts_grouped_product_and_weighted_combine(dtype, n):
    from sglang_security_b200.layers.moe.fused_moe import FusedExperts, TopKRouter
    from sglang_security_b200.layers.scalar_norm import residual_combine

    torch.manual_seed(n)
    width, ff, E, top = 72, 36, 6, 3
    Pw = {"router": torch.randn(E, width).bfloat16(), "router.b": torch.randn(E).bfloat16(),
          "shared.sg": (torch.randn(1, width) / 4).bfloat16()}
    for e in list(range(E)) + ["shared"]:
        k = f"e{e}." if e != "shared" else "shared."
        Pw[k + "gate"], Pw[k + "up"], Pw[k + "down"] = ((torch.randn(ff, width) / 8).bfloat16(),
                                                        (torch.randn(ff, width) / 8).bfloat16(),
                                                        (torch.randn(width, ff) / 6).bfloat16())
    h = torch.randn(n, width).bfloat16()
    want = P.moe_ff(h.double(), {k: v.double() for k, v in Pw.items()},
                    {"router": {"top": top}, "shared": {"ff": ff}})
    router = TopKRouter(width, E, top, True, True).to(DEV)
    router.weight.data.copy_(Pw["router"].float())
    router.bias.data.copy_(Pw["router.b"].float())
    router.shared_gate.data.copy_(Pw["shared.sg"].float().reshape(-1))
    ex = FusedExperts(width, ff, E, "silu", dtype).to(DEV)
    for e in range(E):
        ex.load_expert(e, *(Pw[f"e{e}.{k}"].to(DEV).to(dtype) for k in ("gate", "up", "down")))
    hd = h.to(DEV).to(dtype)
    ids, wts, gate = router(hd)
    rows = ex(hd, ids)
    shared = P.gated_ff(h.double(), Pw["shared.gate"].double(), Pw["shared.up"].double(),
                        Pw["shared.down"].double(), P.silu).to(dtype).to(DEV)
    x = torch.zeros(n, width, device=DEV)
    residual_combine(x, None, None, rows, wts, shared, gate)
    tol = 1e-5 if dtype == torch.float32 else 3e-2
    assert (x.double().cpu() - want).abs().max() <= tol * want.abs().max()


def test_residual_combine_sums_in_fp32():
    from sglang_security_b200.layers.scalar_norm import residual_combine

    x = torch.full((3, 50), 1000.0, device=DEV)
    a = torch.full((3, 50), 0.25, device=DEV, dtype=torch.bfloat16)
    b = torch.full((3, 50), 0.125, device=DEV, dtype=torch.bfloat16)
    residual_combine(x, a, b)
    assert torch.equal(x, torch.full_like(x, 1000.375))     # would be lost in a 16-bit residual


def _attn_setup(m, width, dtype, seed):
    from sglang_security_b200.layers.attention.latent_attention import LatentAttention

    g = torch.Generator().manual_seed(seed)
    H, D = m["heads"], m["dim"] + m["rot_dim"]
    lin = lambda o, i, s=1.0: (torch.randn(o, i, generator=g) * s / i ** 0.5).bfloat16()
    Pw = {"dq": lin(m["q_rank"], width), "dq.norm": (1 + 0.2 * torch.randn(m["q_rank"], generator=g)).bfloat16(),
          "uq": lin(H * D, m["q_rank"], 3.0), "dkv": lin(m["kv_rank"] + m["rot_dim"], width, 2.0),
          "dkv.norm": (1 + 0.2 * torch.randn(m["kv_rank"], generator=g)).bfloat16(),
          "uk": lin(H * m["dim"], m["kv_rank"], 2.0), "uv": lin(H * m["vdim"], m["kv_rank"]),
          "o": lin(width, H * m["vdim"])}
    layer = LatentAttention(width, H, m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"], m["q_rank"], m["scale"],
                            0, 1e-5, window=m.get("mask", {}).get("size"), rope_base=m["rot"]["base"],
                            rope_dims=m["rot"]["dims"], params_dtype=dtype).to(DEV)
    to = lambda t: t.to(DEV).to(dtype)
    layer.load_down(to(Pw["dq"]), to(Pw["dkv"]))
    layer.q_up_proj.weight.data.copy_(to(Pw["uq"]))
    layer.o_proj.weight.data.copy_(to(Pw["o"]))
    layer.load_uk(to(Pw["uk"]))
    layer.load_uv(to(Pw["uv"]))
    layer.q_norm_weight.data.copy_(Pw["dq.norm"].float())
    layer.kv_norm_weight.data.copy_(Pw["dkv.norm"].float())
    return layer, Pw


@pytest.mark.parametrize("dtype,form", [(torch.float32, None), (torch.bfloat16, None),
                                        (torch.bfloat16, "absorbed"), (torch.bfloat16, "expanded"),
                                        (torch.bfloat16, "split")])
@pytest.mark.parametrize("geom", [
    dict(heads=3, dim=24, rot_dim=8, vdim=20, kv_rank=40, q_rank=24, window=9),
    dict(heads=8, dim=16, rot_dim=16, vdim=32, kv_rank=64, q_rank=48, window=33, rot_dims=8),
    dict(heads=1, dim=8, rot_dim=4, vdim=8, kv_rank=24, q_rank=8, window=1),
    dict(heads=10, dim=32, rot_dim=32, vdim=48, kv_rank=160, q_rank=64, window=None),
    dict(heads=5, dim=64, rot_dim=64, vdim=64, kv_rank=288, q_rank=96, window=70),
    dict(heads=2, dim=48, rot_dim=16, vdim=128, kv_rank=72, q_rank=40, window=130),
    dict(heads=2, dim=96, rot_dim=64, vdim=40, kv_rank=64, q_rank=40, window=65),     # no expanded form
])
def test_latent_attention_portions_against_whole_sequence(dtype, form, geom):
    """Portions of unequal size (two requests side by side, one also decoded token by token) against
    the plain attention over the whole sequence: window edges, 32-key tile edges and page edges are
    all crossed; the single tokens of the long request see more than 128 keys where there is no
    window, which is where the 16-bit path spreads a token's keys over several CTAs.  `form` pins
    the absorbed or the expanded form of the sum for every step; "split" takes long portions
    expanded and short ones absorbed inside one step, so both forms meet in one sequence and one
    batch (None: the layer's own choice, which at these sizes is the absorbed form)."""
    import desirax_util as U
    from sglang_security_b200.managers.schedule_batch import Req, StepItem, prepare
    from sglang_security_b200.mem_cache.latent_pool import LatentTokenToKVPool, SeqStatePool
    from sglang_security_b200.mem_cache.memory_pool import ReqToTokenPool
    from sglang_security_b200.mem_cache.paged_allocator import PagedTokenToKVPoolAllocator

    m = U.mixer(**geom)
    width = 56
    layer, Pw = _attn_setup(m, width, dtype, seed=geom["heads"])
    layer.force_form = form
    n = [400, 71]
    g = torch.Generator().manual_seed(3)
    hs = [torch.randn(k, width, generator=g).bfloat16() for k in n]
    Pd = {k: v.double() for k, v in Pw.items()}
    want = []
    for h in hs:
        pos = torch.arange(h.shape[0])
        c, kr = P.latent_kv(h.double(), Pd["dkv"], Pd["dkv.norm"], m["kv_rank"], m["rot"]["base"],
                            m["rot"]["dims"], 1e-5, pos)
        want.append(P.latent_attention(h.double(), c, kr, Pd, m, 1e-5, pos))
    page = 16
    r2t = ReqToTokenPool(3, 512, DEV)
    pool = LatentTokenToKVPool(512, page, dtype, {0: m["kv_rank"] + m["rot_dim"]}, {}, DEV)
    pool.kv_buffer[0].fill_(float("nan"))          # a read of a row that was never written shows
    alloc = PagedTokenToKVPoolAllocator(512, page, dtype, DEV)
    reqs = [Req(rid=str(i), input_ids=[]) for i in range(2)]
    for r in reqs:
        r.req_pool_idx = r2t.alloc(1)[0]
    cuts = [[290, 2, 23, 31, 1, 1, 1, 51], [3, 64, 1, 1, 1, 1]]   # single tokens past 300 keys: split-KV
    got = [[], []]
    at = [0, 0]
    for step in range(max(len(c) for c in cuts)):
        items, who = [], []
        for i in (0, 1):
            if step < len(cuts[i]):
                items.append(StepItem(reqs[i], [0] * cuts[i][step]))
                who.append(i)
        fb = prepare(items, r2t, alloc, pool, SeqStatePool(3, {}, DEV), DEV)
        x = torch.cat([hs[i][at[i]:at[i] + cuts[i][step]] for i in who]).to(DEV).to(dtype)
        out = layer(x, fb).double().cpu()
        o = 0
        for i in who:
            got[i].append(out[o:o + cuts[i][step]])
            o += cuts[i][step]
            at[i] += cuts[i][step]
    tol = 2e-5 if dtype == torch.float32 else 4e-2
    for i in (0, 1):
        assert at[i] == n[i]
        res = torch.cat(got[i])
        assert torch.isfinite(res).all()
        assert (res - want[i]).abs().max() <= tol * want[i].abs().max(), (i, (res - want[i]).abs().max())
