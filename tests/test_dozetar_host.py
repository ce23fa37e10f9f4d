"""Dozetar, host side (no GPU): configuration reader, registry, tensor-name mapping, and self-checks
of the plain restatement the GPU tests compare against."""
import pytest
import torch

import dozetar_plain as P
import dozetar_util as U


def _cfg():
    return U.config([(U.mlstm(), U.experts(5, 2, 24)), (U.parallel(), U.experts(4, 1, 16)), (U.mlstm(2, 8, 12), None)])


def test_config_reads_every_size_and_constant():
    from sglang_security_b200.configs.dozetar import dozetar_config

    raw = _cfg()
    c = dozetar_config(raw)
    assert (c.vocab, c.width, c.eps, c.residual_mult, c.logit_softcap) == (97, 40, 1e-5, 0.6, 20.0)
    assert [L.type for L in c.layers] == ["mlstm", "parallel", "mlstm"]
    a = c.layers[1].mixer
    assert (a.left.heads, a.left.kv_heads, a.left.dim, a.left.vdim) == (4, 2, 16, 24)
    assert (a.left.window, a.left.keep_first, a.left.rope_dims, a.left.rope_base) == (9, 2, 8, 1000.0)
    assert a.right.decay == raw["layers"][1]["mixer"]["right"]["decay"] and a.left_scale == 0.7
    assert c.layers[0].mlp.top == 2 and c.layers[2].mlp is None and c.layers[0].mixer.gate_cap == 8.0


def test_config_defaults_and_rejections():
    from sglang_security_b200.configs.dozetar import dozetar_config

    raw = U.config([(U.parallel(window=None, rot_dims=0), None)], softcap=None)
    c = dozetar_config(raw)
    assert c.logit_softcap == 0.0 and c.layers[0].mixer.left.window is None
    assert c.layers[0].mixer.left.rope_dims == 0 and c.layers[0].mixer.left.keep_first == 0
    bad = U.config([(U.parallel(heads=3, kv_heads=2), None)])
    with pytest.raises(ValueError):
        dozetar_config(bad)
    bad = U.config([(U.parallel(rot_dims=18, dim=16), None)])
    with pytest.raises(ValueError):
        dozetar_config(bad)
    bad = U.config([(dict(U.mlstm(), type="conv"), None)])
    with pytest.raises(ValueError):
        dozetar_config(bad)
    bad = U.config([(U.mlstm(), U.experts(3, 4, 8))])
    with pytest.raises(ValueError):
        dozetar_config(bad)


def test_model_config_picks_the_design(tmp_path):
    from sglang_security_b200.configs.dozetar import DozetarConfig
    from sglang_security_b200.configs.model_config import ModelConfig
    from sglang_security_b200.models.registry import resolve_model_cls, supported_architectures

    cfg = _cfg()
    folder = U.write_model(str(tmp_path / "m"), cfg, U.random_weights(cfg))
    mc = ModelConfig(folder)
    assert mc.architecture == "Dozetar" and isinstance(mc.hf_config, DozetarConfig)
    assert {"Desirax", "Dozetar"} <= set(supported_architectures())
    assert resolve_model_cls("Dozetar").__name__ == "DozetarForCausalLM"


def test_expected_tensor_names_match_the_weights():
    from sglang_security_b200.configs.dozetar import dozetar_config
    from sglang_security_b200.models.dozetar import DozetarForCausalLM

    cfg = _cfg()
    model = DozetarForCausalLM.__new__(DozetarForCausalLM)
    model.config = dozetar_config(cfg)
    assert DozetarForCausalLM.expected_tensor_names(model) == set(U.random_weights(cfg))


def test_plain_window_keeps_first_tokens():
    ok = P.visible(12, 4, 2)
    assert ok[10].nonzero().flatten().tolist() == [0, 1, 7, 8, 9, 10]
    assert ok[3].nonzero().flatten().tolist() == [0, 1, 2, 3]
    assert P.visible(5, None, 0)[4].all()


def test_plain_gated_recurrence_equals_the_unstabilised_sums():
    """The stabiliser only rescales numerator and denominator: running the recurrence with the exact
    un-stabilised sums gives the same outputs."""
    g = torch.Generator().manual_seed(3)
    T, H, D, E = 9, 2, 4, 3
    q, k = torch.randn(T, H, D, generator=g, dtype=P.DT), torch.randn(T, H, D, generator=g, dtype=P.DT)
    v = torch.randn(T, H, E, generator=g, dtype=P.DT)
    li, lf = torch.randn(T, H, generator=g, dtype=P.DT), -torch.rand(T, H, generator=g, dtype=P.DT)
    out = P.mlstm_recurrence(q, k, v, li, lf)
    F = torch.cumsum(lf, 0)
    for t in range(T):
        for h in range(H):
            wts = torch.exp(F[t, h] - F[:t + 1, h] + li[:t + 1, h])
            num = (wts[:, None] * (k[:t + 1, h] @ q[t, h])[:, None] * v[:t + 1, h]).sum(0)
            den = (wts * (k[:t + 1, h] @ q[t, h])).sum()
            m = torch.maximum(F[t, h], (F[t, h] - F[:t + 1, h] + li[:t + 1, h]).max())
            want = num / (torch.maximum(den.abs(), torch.tensor(1.0, dtype=P.DT)) + 1e-6 * torch.exp(m))
            assert torch.allclose(out[t, h], want, rtol=1e-9, atol=1e-12)


def test_plain_sink_only_shrinks_the_weights():
    g = torch.Generator().manual_seed(4)
    q, k, v = (torch.randn(6, 2, 4, generator=g, dtype=P.DT) for _ in range(3))
    a = P.sink_softmax(q, k, v, 0.5, None, 0, None)
    b = P.sink_softmax(q, k, v, 0.5, None, 0, torch.full((2,), -60.0, dtype=P.DT))
    c = P.sink_softmax(q, k, v, 0.5, None, 0, torch.full((2,), 60.0, dtype=P.DT))
    assert torch.allclose(a, b) and c.abs().max() < 1e-15 * 1e6
