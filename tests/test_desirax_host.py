"""Host-side parts of the Desirax path that need no GPU: configuration reader, model registry,
safetensors reader, scheduler policy (against a stand-in runner), and sanity of the plain oracle."""
import json
import math

import pytest
import torch

import desirax_plain as P
import desirax_util as U


def test_config_reader_takes_every_size_from_the_file(tmp_path):
    from sglang_security_b200.configs.model_config import ModelConfig

    cfg = U.config([(U.mixer(heads=5, dim=12, rot_dim=6, vdim=7, kv_rank=44, q_rank=20, window=13, base=123.0,
                             scale=0.37), U.moe(11, 3, 28, 60)),
                    (U.mixer(heads=5, dim=12, rot_dim=6, vdim=9, kv_rank=44, q_rank=10, window=None, base=123.0,
                             kv_from=0), None)], vocab=211, width=52, eps=3e-4)
    folder = U.write_model(str(tmp_path / "m"), cfg, {})
    mc = ModelConfig(folder)
    c = mc.hf_config
    assert mc.architecture == "Desirax" and (c.vocab, c.width, c.eps) == (211, 52, 3e-4)
    m0, m1 = c.layers[0].mixer, c.layers[1].mixer
    assert (m0.heads, m0.dim, m0.rot_dim, m0.vdim, m0.kv_rank, m0.q_rank, m0.window, m0.rope_base, m0.scale,
            m0.rope_dims, m0.kv_from) == (5, 12, 6, 7, 44, 20, 13, 123.0, 0.37, 6, None)
    assert m1.window is None and m1.kv_from == 0 and c.layers[1].mlp is None
    f = c.layers[0].mlp
    assert (f.kind, f.experts, f.top, f.expert_ff, f.shared_ff, f.act) == ("moe", 11, 3, 28, 60, "silu")


@pytest.mark.parametrize("bad", ["forward", "chain", "sizes", "type"])
def test_config_reader_rejects_inconsistent_layers(bad):
    from sglang_security_b200.configs.desirax import desirax_config

    layers = [(U.mixer(), U.dense()), (U.mixer(kv_from=0), None), (U.mixer(), None)]
    if bad == "forward":
        layers[1] = (U.mixer(kv_from=2), None)
    elif bad == "chain":
        layers[2] = (U.mixer(kv_from=1), None)
    elif bad == "sizes":
        layers[1] = (U.mixer(kv_from=0, kv_rank=48), None)
    cfg = U.config(layers)
    if bad == "type":
        cfg["layers"][0]["type"] = "something_else"
    with pytest.raises(ValueError):
        desirax_config(cfg)


def test_registry_resolves_by_architecture_name():
    from sglang_security_b200.models.registry import resolve_model_cls, supported_architectures

    assert "Desirax" in supported_architectures()
    assert resolve_model_cls("Desirax").__name__ == "DesiraxForCausalLM"
    with pytest.raises(ValueError):
        resolve_model_cls("NoSuchModel")


def test_safetensors_reader_round_trip_and_model_loading_on_cpu(tmp_path):
    from sglang_security_b200.configs.model_config import ModelConfig
    from sglang_security_b200.model_loader.safetensors_reader import SafetensorsFile
    from sglang_security_b200.models.registry import resolve_model_cls

    cfg = U.config([(U.mixer(), U.dense()), (U.mixer(kv_from=0), U.moe())])
    w = U.random_weights(cfg, 1)
    w["table"] = torch.arange(6, dtype=torch.int32).reshape(2, 3)
    folder = U.write_model(str(tmp_path / "m"), cfg, w)
    f = SafetensorsFile(folder + "/model.safetensors")
    assert set(f.keys()) == set(w)
    for k, t in w.items():
        got = f.get(k)
        assert got.dtype == t.dtype and got.shape == t.shape and torch.equal(got, t)
    del w["table"]
    mc = ModelConfig(folder)
    model = resolve_model_cls(mc.architecture)(mc.hf_config, torch.bfloat16)
    model.load_weights(w.items())
    L1 = model.layers[1]
    assert torch.equal(L1.mix.down_proj.weight, w["l1.mix.dq"])          # no KV projection of its own
    assert torch.equal(model.layers[0].mix.down_proj.weight, torch.cat([w["l0.mix.dq"], w["l0.mix.dkv"]]))
    assert torch.equal(L1.moe.experts.w_gate_up[3, :24], w["l1.mlp.e3.gate"])
    assert torch.equal(L1.moe.experts.w_gate_up[3, 24:], w["l1.mlp.e3.up"])
    assert torch.equal(model.layers[0].mix.w_uv_t[2], w["l0.mix.uv"].view(3, 20, 40)[2].T)
    assert float(model.layers[0].norm1.gain) == float(w["l0.norm1"])
    spec = model.cache_spec()
    assert spec.row_dims == {0: 48} and spec.source_of == {1: 0} and spec.state_widths == {0: 40, 1: 40}
    missing = dict(w)
    del missing["l1.mlp.e2.up"]
    with pytest.raises(ValueError):
        resolve_model_cls(mc.architecture)(mc.hf_config, torch.bfloat16).load_weights(missing.items())
    with pytest.raises(ValueError):
        model.load_weights(list(w.items()) + [("l0.mix.extra", torch.zeros(1))])


class _FakeRunner:
    """Counts pages like ModelRunner, runs nothing."""
    device, page_size = "cpu", 64

    def __init__(self, pages=8, slots=4):
        self.max_total_tokens = self.context_length = pages * 64
        self.free_pages, self.slots, self.log = pages, slots, []

    def admit(self, req):
        if not self.slots:
            return False
        self.slots -= 1
        req.req_pool_idx, req.cached_len = 0, 0
        return True

    def release(self, req):
        self.free_pages += (req.cached_len + 63) // 64
        self.slots += 1

    def free_token_slots(self):
        return self.free_pages * 64

    def forward(self, items, layer_hook=None):
        self.log.append([(it.req.rid, len(it.tokens), list(it.want)) for it in items])
        for it in items:
            before = (it.req.cached_len + 63) // 64
            it.req.cached_len += len(it.tokens)
            self.free_pages -= (it.req.cached_len + 63) // 64 - before
            assert self.free_pages >= 0
        rows = sum(len(it.want) for it in items)
        out = torch.zeros(rows, 10)
        out[:, 3] = 1.0
        return out


def test_scheduler_chunks_prompts_mixes_decodes_and_respects_slots_and_pages():
    from sglang_security_b200.managers.schedule_batch import Req, SamplingParams
    from sglang_security_b200.managers.scheduler import Scheduler

    run = _FakeRunner(pages=8, slots=2)
    s = Scheduler(run, chunked_prefill_size=100)
    s.sampler = type("S", (), {"__call__": lambda self, logits, reqs: [3] * len(reqs),
                             "forget": lambda self, rid: None})()
    sp = SamplingParams(max_new_tokens=3)
    for rid, n in (("a", 150), ("b", 30), ("c", 200)):
        s.add_request(Req(rid=rid, input_ids=[1] * n,
                          sampling_params=SamplingParams(max_new_tokens=8) if rid == "b" else sp))
    done = []
    for _ in range(40):
        done += [r.rid for r in s.step()]
        if s.idle():
            break
    assert s.idle() and sorted(done) == ["a", "b", "c"]
    assert run.free_pages == 8 and run.slots == 2
    log = run.log
    assert log[0] == [("a", 100, [])]                                  # the budget cuts the prompt
    assert log[1] == [("a", 50, [49]), ("b", 30, [29])]                # rest of a, then the next request
    assert log[2] == [("a", 1, [0]), ("b", 1, [0])]                    # c waits: both slots are taken
    assert any(("c", 100, []) in st and any(e[1] == 1 for e in st) for st in log)   # prompt beside decodes
    assert all(sum(n for _, n, _ in st if n > 1) <= 100 for st in log)
    with pytest.raises(ValueError):
        s.add_request(Req(rid="big", input_ids=[1] * 600, sampling_params=sp))


def test_plain_oracle_token_shift_rotation_and_window():
    h = torch.arange(12.0).reshape(4, 3)
    mu = torch.tensor([0.0, 1.0, 0.5])
    out = P.token_shift(h, mu)
    assert torch.equal(out[:, 0], h[:, 0])                              # mu 0: the token itself
    assert torch.equal(out[1:, 1], h[:-1, 1]) and out[0, 1] == 0        # mu 1: the previous token, zeros first
    v = torch.randn(5, 2, 6, dtype=torch.float64)
    pos = torch.arange(5)
    r = P.rotate_interleaved(v, pos, 100.0, 4)
    assert torch.equal(r[..., 4:], v[..., 4:]) and torch.allclose(r[0], v[0])
    assert torch.allclose(r[..., :4].norm(dim=-1), v[..., :4].norm(dim=-1))
    a = 3 * 100.0 ** (-2 / 4)
    assert math.isclose(float(r[3, 1, 2]), float(v[3, 1, 2] * math.cos(a) - v[3, 1, 3] * math.sin(a)), rel_tol=1e-12)
    # window w: the output at i must not change when a token w or more back changes
    cfg = U.config([(U.mixer(window=4), None)])
    w = U.random_weights(cfg, 0)
    t1 = [1, 2, 3, 4, 5, 6, 7, 8]
    t2 = [9] + t1[1:]
    l1, l2 = P.forward(cfg, w, t1), P.forward(cfg, w, t2)
    # token 0 reaches position i through the shift (i = 1) and the window (i <= 3) only
    assert not torch.allclose(l1[3], l2[3]) and torch.allclose(l1[5:], l2[5:])


def test_expanded_attention_plan_tables_and_choice():
    """Host side of the expanded attention form: which steps take it, and the gather tables (first
    gathered key of every request = its window's lower edge, positions shifted to start there)."""
    from types import SimpleNamespace

    import torch

    from sglang_security_b200.layers.attention.latent_attention import LatentAttention, _visible_pairs

    # (query, key) pairs under a causal window, against the count done by hand
    for prefix, new, window in [(0, 5, 3), (10, 4, 0), (1, 4, 4), (7, 1, 2), (0, 1, 1), (3, 9, 100)]:
        want = sum(min(prefix + i + 1, window) if window else prefix + i + 1 for i in range(new))
        assert _visible_pairs(prefix, new, window) == want
    layer = LatentAttention(64, heads=4, dim=24, rot_dim=8, vdim=40, kv_rank=256, q_rank=32, scale=0.2,
                            layer_id=0, eps=1e-5, window=60, params_dtype=torch.bfloat16)
    assert layer.expand_dim == 64
    big = LatentAttention(64, heads=2, dim=96, rot_dim=64, vdim=40, kv_rank=48, q_rank=32, scale=0.2,
                          layer_id=0, eps=1e-5, window=10, params_dtype=torch.bfloat16)
    assert big.expand_dim == 0                      # heads wider than 128: no expanded form
    r2t = torch.arange(3 * 2100, dtype=torch.int32).view(3, 2100) + 1000

    def batch(pre, ext, rows, row_dim=256 + 8):
        start = [sum(ext[:b]) for b in range(len(ext))]
        pool = SimpleNamespace(get_kv_buffer=lambda layer_id: torch.zeros(4, row_dim, dtype=torch.bfloat16))
        return SimpleNamespace(extend_prefix_lens_cpu=pre, extend_seq_lens_cpu=ext, extra={},
                               req_pool_indices=torch.tensor(rows, dtype=torch.int64),
                               req_to_token_pool=SimpleNamespace(req_to_token=r2t), token_to_kv_pool=pool,
                               ext_len=torch.tensor(ext, dtype=torch.int32),
                               ext_start=torch.tensor(start, dtype=torch.int32),
                               tok_b=torch.repeat_interleave(torch.arange(len(ext), dtype=torch.int32),
                                                             torch.tensor(ext)))

    assert layer._expand_plan(batch([50, 60], [1, 1], [0, 1])) is False          # decoding stays absorbed
    tiny = LatentAttention(64, heads=4, dim=24, rot_dim=8, vdim=40, kv_rank=48, q_rank=32, scale=0.2,
                           layer_id=0, eps=1e-5, window=4, params_dtype=torch.bfloat16)
    assert tiny._expand_plan(batch([0], [100], [0], 56)) is False                # so does a tiny window
    assert big._expand_plan(batch([0], [150], [0])) is False
    # at these sizes the saving is below the fixed cost of the expanded form's extra launches
    assert layer._expand_plan(batch([0, 90], [100, 64], [2, 0])) is False
    wide = LatentAttention(64, heads=16, dim=64, rot_dim=64, vdim=128, kv_rank=512, q_rank=32, scale=0.2,
                           layer_id=0, eps=1e-5, window=4096, params_dtype=torch.bfloat16)
    assert wide._expand_plan(batch([0], [2048], [0], 576))["rest"] is None       # a long prompt: expanded
    assert wide._expand_plan(batch([0, 150], [40, 1], [0, 1], 576)) is False     # a short one beside a decode: not
    # a divided step: two long portions expanded, a decoded token and a 3-token portion absorbed
    layer.force_form = "split"
    fb = batch([0, 150, 90, 4], [100, 1, 64, 3], [2, 1, 0, 1])
    plan = layer._expand_plan(fb)
    assert plan and layer._expand_plan(fb) is plan                               # one plan per step
    lo = [0, 31]                                    # 90 - 60 + 1 = 31: the first key the portion's first token sees
    n = [100, 90 + 64 - 31]
    assert plan["N"] == sum(n) and plan["max_ext"] == 100 and plan["bs"] == 2
    assert plan["prefix"].tolist() == [0, 59] and plan["seq"].tolist() == n
    assert plan["ext_len"].tolist() == [100, 64] and plan["ext_start"].tolist() == [0, 101]
    want_slots = torch.cat([r2t[row, l:l + k] for row, l, k in zip([2, 0], lo, n)]).long()
    assert torch.equal(plan["slots"], want_slots)
    off = [0, n[0]]
    for b in range(2):
        assert plan["rtt"][b, :n[b]].tolist() == list(range(off[b], off[b] + n[b]))
    rest = plan["rest"]
    assert rest["bs"] == 2 and rest["tokens"] == 4 and rest["max_seq"] == 151
    assert rest["ext_len"].tolist() == [1, 3] and rest["ext_start"].tolist() == [100, 165]
    assert rest["req_pool"].tolist() == [1, 1]
    assert plan["tok_mask"].tolist() == [True] * 100 + [False] + [True] * 64 + [False] * 3
    # all entries long: nothing is left for the absorbed form
    whole = layer._expand_plan(batch([0, 90], [100, 64], [2, 0]))
    assert whole and whole["rest"] is None and whole["bs"] == 2
    # a latent the tiled absorbed kernel does not take (rank not a multiple of 8): the step is not divided
    odd = LatentAttention(64, heads=4, dim=24, rot_dim=8, vdim=40, kv_rank=252, q_rank=32, scale=0.2,
                          layer_id=0, eps=1e-5, window=60, params_dtype=torch.bfloat16)
    odd.force_form = "split"
    p2 = odd._expand_plan(batch([0, 150, 90, 4], [100, 1, 64, 3], [2, 1, 0, 1], 260))
    assert p2 is False or p2["rest"] is None
    layer.force_form = "absorbed"
    assert layer._expand_plan(batch([0], [150], [0])) is False
    layer.force_form = "expanded"
    assert layer._expand_plan(batch([50], [1], [0]))
