"""CPU: the host side of the Nirelix decoder -- registry and native configuration, presets, checkpoint tensors routed
onto fused and padded parameters (inner sizes of the low-rank projections taken from the tensors' shapes), the padded
merged projection, and the float64 oracle's own invariants (so that the GPU tests compare against something sound)."""
import json
import math

import pytest
import torch

import nirelix_oracle as O
from test_nirelix_gpu import config_a, config_b, config_c

F64 = torch.float64


def test_registry_native_config_and_presets(tmp_path):
    from nanovllm.config import Config, NativeConfig
    from nanovllm.models.models_map import model_dict
    from nanovllm.engine.model_runner import _resolve_dtype
    cfg = config_a()
    with open(tmp_path / "config.json", "w") as f:
        json.dump(cfg, f)
    c = Config(str(tmp_path), max_model_len=64, max_num_batched_tokens=64, dtype="float32")
    assert isinstance(c.hf_config, NativeConfig) and c.hf_config.architectures == ["Nirelix"]
    assert model_dict["Nirelix"].supports_fp32 and not model_dict["Nirelix"].prefix_caching
    assert _resolve_dtype(c.hf_config, "float32", model_dict["Nirelix"]) == torch.float32
    p = Config("tiny-nirelix").hf_config.to_dict()
    assert [l["type"] for l in p["layers"]] == ["retention", "channel_delta", "latent_attention"] and p["streams"] == 2
    big = Config("nirelix-1k").hf_config.to_dict()
    assert len(big["layers"]) == 28 and big["width"] == 1024


@pytest.mark.parametrize("make,ranks", [(config_a, (5, 3)), (config_b, (8, 16)), (config_c, (7, 2))])
def test_checkpoint_tensors_route_onto_the_model(tmp_path, make, ranks):
    """Every tensor of a checkpoint lands somewhere, every parameter is covered, fused projections hold the pieces in
    the order the mixers slice them, and padding rows and columns stay zero."""
    from safetensors.torch import save_file
    from nanovllm.config import NativeConfig
    from nanovllm.layers.moe import GroupedSigmoidMoe
    from nanovllm.models.models_map import model_dict
    from nanovllm.utils.loader import checkpoint_shapes, load_model
    cfg = make()
    tensors = O.random_model(cfg, seed=3, ranks=ranks)
    save_file({k: v.contiguous() for k, v in tensors.items()}, str(tmp_path / "model.safetensors"))
    native = NativeConfig(cfg)
    native.checkpoint_shapes = checkpoint_shapes(str(tmp_path))
    assert native.checkpoint_shapes["embed"] == (cfg["vocab"], cfg["width"])
    model = model_dict["Nirelix"](native)
    padded = {"small.weight", "a_up.weight", "g_up.weight", "mix.proj.weight"}
    unit = {f"layers.{i}.mix.norm.weight" for i, e in enumerate(cfg["layers"]) if e["type"] == "retention"}
    for n, p in model.named_parameters():                    # all but zero padding and weights that no tensor fills
        if not any(n.endswith(s) for s in padded) and not ("hc" in n and "streams" not in cfg) and n not in unit:
            p.data.fill_(float("nan"))
    assert load_model(model, str(tmp_path)) == len(tensors)
    assert not any(torch.isnan(p).any() for p in model.parameters())
    for i, entry in enumerate(cfg["layers"]):
        layer, mix, m = model.layers[i], model.layers[i].mix, entry["mixer"]
        t = lambda n: tensors[f"l{i}.{n}"].float()
        assert torch.equal(layer.norm1.weight, t("norm1")) and torch.equal(layer.norm1.bias, t("norm1.b"))
        if "streams" in cfg:
            assert torch.equal(layer.hc1.read, t("hc1.in")) and torch.equal(layer.hc1.write, t("hc1.out"))
            assert torch.equal(layer.hc1.mix, t("hc1.mix"))
        else:
            assert torch.equal(layer.hc1.mix, torch.eye(1)) and float(layer.hc1.read) == 1.0
        if entry["type"] == "retention":
            nq, nv = m["heads"] * m["dim"], m["heads"] * m["vdim"]
            w = mix.proj.weight.float()
            assert torch.equal(w[:nq], t("mix.q")) and torch.equal(w[nq:2 * nq], t("mix.k"))
            assert torch.equal(w[2 * nq:2 * nq + nv], t("mix.v")) and torch.equal(w[2 * nq + nv:], t("mix.g"))
            assert torch.allclose(mix.rec.decay, torch.tensor(m["decay"])) and float(mix.norm.weight.min()) == 1.0
        elif entry["type"] == "channel_delta":
            H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
            w = mix.proj.weight.float()
            assert torch.equal(w[G * d:2 * G * d], t("mix.k")) and torch.equal(w[2 * G * d:], t("mix.v"))
            assert torch.equal(mix.conv.weight[2 * G * d:], t("mix.v.conv"))
            s = mix.small
            assert s.output_sizes == [ranks[0], ranks[1], H] and all(n % 8 == 0 for n in s.padded_sizes)
            y = torch.arange(s.weight.shape[0], dtype=torch.float32)[None]
            rows = lambda part: s.part(y, part)[0].long()
            assert torch.equal(s.weight.float()[rows(0)], t("mix.a1")) and torch.equal(s.weight.float()[rows(2)], t("mix.b"))
            assert float(s.weight.float().abs().sum()) == pytest.approx(
                float(t("mix.a1").abs().sum() + t("mix.g1").abs().sum() + t("mix.b").abs().sum()), rel=1e-5)
            assert torch.equal(mix.a_up.weight.float()[:H * d, :ranks[0]], t("mix.a2"))
            assert not mix.a_up.weight[:, ranks[0]:].any()
            assert torch.equal(mix.norm.weight, t("mix.norm").repeat(H)) and torch.equal(mix.rule.dt_bias, t("mix.dt_bias"))
        else:
            H, d, dr, R, Q = m["heads"], m["dim"], m["rot_dim"], m["kv_rank"], m["q_rank"]
            y = torch.arange(mix.proj.weight.shape[0], dtype=torch.float32)[None]
            assert torch.equal(mix.proj.weight.float()[mix.proj.part(y, 1)[0].long()], t("mix.dkv"))
            assert torch.equal(mix.attn.w_uk.float().reshape(H * d, R), t("mix.uk"))
            assert torch.equal(mix.attn.w_uv.float()[1], t("mix.uv")[m["vdim"]:2 * m["vdim"]])
            assert torch.equal(mix.kv_norm, t("mix.dkv.norm")) and mix.attn.window == (m.get("mask") or {}).get("size", 0)
        if isinstance(layer.mlp, GroupedSigmoidMoe):
            ff, e = entry["mlp"]["expert"]["ff"], entry["mlp"]["router"]["experts"] - 1
            assert torch.equal(layer.mlp.w13.float()[e, ff:], t(f"mlp.e{e}.up")) and layer.mlp.router.dtype == torch.float32
            assert torch.equal(layer.mlp.w2.float()[0], t("mlp.e0.down")) and torch.equal(layer.mlp.correction, t("mlp.correction"))
        elif layer.mlp is not None:
            assert torch.equal(layer.mlp.gate_up_proj.weight.float()[entry["mlp"]["ff"]:], t("mlp.up"))
            assert layer.mlp.limit == entry["mlp"]["limit"]
    assert torch.equal(model.lm_head.weight.float(), tensors["head"].float())
    assert torch.equal(model.norm.bias, tensors["final.norm.b"].float())


def test_random_init_keeps_padding_zero():
    from nanovllm.config import Config
    from nanovllm.models.models_map import model_dict
    model = model_dict["Nirelix"](Config("tiny-nirelix").hf_config)
    model.random_init(1)
    delta = model.layers[1].mix
    assert not delta.small.weight[delta.small.output_sizes[0]:delta.small.padded_sizes[0]].any()
    assert torch.equal(delta.norm.weight[:delta.dv], delta.norm.weight[delta.dv:2 * delta.dv])
    assert all(torch.isfinite(p).all() for p in model.parameters())


# ------------------------------------------------------------------ the oracle's own invariants
def test_oracle_rotation_is_relative_and_layouts_differ():
    g = torch.Generator().manual_seed(0)
    q, k = torch.randn(1, 1, 8, generator=g, dtype=F64), torch.randn(1, 1, 8, generator=g, dtype=F64)
    for inter in (False, True):
        a = (O.rotate(q, torch.tensor([7]), 6, 100.0, inter) * O.rotate(k, torch.tensor([3]), 6, 100.0, inter)).sum()
        b = (O.rotate(q, torch.tensor([104]), 6, 100.0, inter) * O.rotate(k, torch.tensor([100]), 6, 100.0, inter)).sum()
        assert abs(float(a - b)) < 1e-9
        assert torch.equal(O.rotate(q, torch.tensor([5]), 6, 100.0, inter)[..., 6:], q[..., 6:])
    assert not torch.allclose(O.rotate(q, torch.tensor([5]), 6, 100.0, True), O.rotate(q, torch.tensor([5]), 6, 100.0, False))


def test_oracle_window_and_delta_rule():
    cfg = config_a()
    t = O.as_f64(O.random_model(cfg, 1))
    toks = list(range(40))
    full = O.forward(cfg, t, toks)
    assert torch.allclose(O.forward(cfg, t, toks[:25]), full[:25], atol=1e-9)       # causal
    m = dict(cfg["layers"][2]["mixer"])
    u = torch.randn(30, cfg["width"], generator=torch.Generator().manual_seed(2), dtype=F64)
    P = O.sub(t, "l2.mix.")
    base = O.latent_attention_mixer(u, P, m, 1e-5)
    u2 = u.clone()
    u2[3] += 1.0                                        # a key outside the window of the last token (19), inside of token 21
    moved = O.latent_attention_mixer(u2, P, m, 1e-5)
    assert torch.allclose(moved[22:], base[22:], atol=1e-12) and not torch.allclose(moved[21], base[21], atol=1e-9)
    # delta rule: with beta = 1 and no decay, writing key e0 twice leaves the second value
    k = torch.zeros(2, 1, 4, dtype=F64)
    k[:, 0, 0] = 1
    v = torch.tensor([[[1.0, 2.0]], [[5.0, -1.0]]], dtype=F64)
    o = O.delta_recurrence(k, k, v, torch.ones(2, 1, 4, dtype=F64), torch.ones(2, 1, dtype=F64))
    assert torch.allclose(o[1, 0], v[1, 0])


def test_oracle_router_groups():
    z = torch.tensor([[4.0, 3.9, -9.0, -9.0, 2.0, 2.0]], dtype=F64)
    corr = torch.tensor([-3.0, -3.0, 0.0, 0.0, 0.0, 0.0], dtype=F64)
    r = {"experts": 6, "top": 2, "groups": {"count": 3, "keep": 1}, "scale": 2.0}
    idx, w = O.route(z, corr, r)                        # group 0 has the largest scores but loses after the correction
    assert sorted(idx[0].tolist()) == [4, 5] and abs(float(w.sum()) - 2.0) < 1e-12
    idx, w = O.route(z, torch.zeros(6, dtype=F64), r)
    assert sorted(idx[0].tolist()) == [0, 1]
    s = torch.sigmoid(z[0, :2])
    assert torch.allclose(w[0].sort().values, (s / s.sum() * 2.0).sort().values)
