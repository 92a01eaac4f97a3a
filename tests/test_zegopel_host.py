"""CPU tests of what the hybrid decoders add to the host side: state slots and the prefix-cache switch of the
block manager, steps over given tokens in the scheduler, the native config reader, and the routing of
checkpoint tensors onto the model's (fused) parameters."""
import json
import os
from types import SimpleNamespace

import pytest
import torch

import zegopel_oracle as O
from test_zegopel_gpu import config_a, config_b


def _sched(blocks=8, block_size=16, seqs=3):
    from nanovllm.engine.scheduler import Scheduler
    cfg = SimpleNamespace(max_num_seqs=seqs, max_num_batched_tokens=4096, max_model_len=blocks * block_size, eos=-1,
                          chunked_prefill=True, num_kvcache_blocks=blocks + 1, kvcache_block_size=block_size,
                          num_state_slots=seqs, enable_prefix_caching=False)
    return Scheduler(cfg)


def test_state_slots_follow_the_blocks():
    from nanovllm.engine.block_manager import BlockManager
    from nanovllm.engine.sequence import Sequence
    bm = BlockManager(6, 4, num_state_slots=2, prefix_caching=False)
    a, b, c = (Sequence(list(range(n)), block_size=4) for n in (9, 4, 3))
    bm.allocate(a)
    bm.allocate(b)
    assert {a.state_slot, b.state_slot} == {0, 1} and len(a.block_table) == 3 and len(b.block_table) == 1
    assert not bm.can_allocate(c)                        # blocks are left, slots are not
    bm.deallocate(a)
    assert a.state_slot == -1 and bm.can_allocate(c)
    bm.allocate(c)
    assert c.state_slot == 0                             # the slot a gave back
    # identical tokens never share blocks without the prefix cache
    d = Sequence(list(range(4)), block_size=4)
    bm.deallocate(c)
    bm.allocate(d)
    assert not set(d.block_table) & set(b.block_table) and d.num_cached_tokens == 0
    # growth: a block when the newest token opened one, nothing registered when one filled
    b.append_token(7)
    bm.may_append(b)
    assert len(b.block_table) == 2 and not bm.hash_to_block_id


def test_given_steps_classify_and_release():
    s = _sched()
    batch, prefill = s.schedule_given([("x", [1, 2, 3, 4, 5]), ("y", [9])])
    assert prefill and [q.prefill_window for q in batch] == [(0, 5), (0, 1)]     # a first token is a prompt
    s.postprocess_given(batch)
    batch, prefill = s.schedule_given([("x", [6]), ("y", [8])])
    assert not prefill and all(q.prefill_window is None for q in batch)          # single tokens of running requests
    assert [len(q) for q in batch] == [6, 2] and [q.last_token for q in batch] == [6, 8]
    s.postprocess_given(batch)
    batch, prefill = s.schedule_given([("x", [7]), ("y", list(range(20)))])
    assert prefill and [q.prefill_window for q in batch] == [(6, 7), (2, 22)]    # a token beside a portion
    assert len(batch[1].block_table) == 2
    s.postprocess_given(batch)
    s.finish_given("y")
    bm = s.block_manager
    assert len(bm.free_state_slots) == 2 and len(bm.free_block_ids) == 7 and "y" not in s.given
    batch, _ = s.schedule_given([("z", [1] * 40)])
    assert batch[0].state_slot == 2                      # slots go round: the one y gave back comes last
    s.postprocess_given(batch)
    with pytest.raises(RuntimeError):
        s.schedule_given([("w", [1] * 100)])             # 7 blocks wanted, 4 of 8 are left
    assert list(bm.free_state_slots) == [1] and len(bm.free_block_ids) == 4      # the refusal took nothing
    batch, _ = s.schedule_given([("v", [2, 3])])
    assert batch[0].state_slot == 1


def test_native_config_and_presets(tmp_path):
    from nanovllm.config import Config, NativeConfig
    cfg = config_a()
    with open(tmp_path / "config.json", "w") as f:
        json.dump(cfg, f)
    c = Config(str(tmp_path), max_model_len=64, max_num_batched_tokens=64, dtype="float32")
    assert isinstance(c.hf_config, NativeConfig) and c.hf_config.architectures == ["Zegopel"]
    assert c.hf_config.to_dict()["layers"][1]["mixer"]["q_temp"]["every"] == 8 and c.eos == -1
    p = Config("tiny-zegopel").hf_config.to_dict()
    assert [l["type"] for l in p["layers"]] == ["attention", "lightning", "mamba2"]


@pytest.mark.parametrize("make", [config_a, config_b])
def test_checkpoint_tensors_route_onto_the_model(tmp_path, make):
    """Every tensor of a checkpoint lands somewhere, every parameter is covered, and the fused projections hold
    the pieces in the order the mixers slice them."""
    from safetensors.torch import save_file
    from nanovllm.config import NativeConfig
    from nanovllm.models.models_map import model_dict
    from nanovllm.utils.loader import load_model
    cfg = make()
    tensors = O.random_model(cfg, seed=3)
    save_file({k: v.contiguous() for k, v in tensors.items()}, str(tmp_path / "model.safetensors"))
    model = model_dict["Zegopel"](NativeConfig(cfg))
    for p in model.parameters():
        p.data.fill_(float("nan"))
    for layer in model.layers:
        if getattr(layer.mix, "proj", None) is not None and layer.mix.proj.bias is not None:
            layer.mix.proj.bias.data.zero_()
    assert load_model(model, str(tmp_path)) == len(tensors)
    assert not any(torch.isnan(p).any() for p in model.parameters())
    for i, entry in enumerate(cfg["layers"]):
        mix, m = model.layers[i].mix, entry["mixer"]
        t = lambda n: tensors[f"l{i}.mix.{n}"].float()
        if entry["type"] == "attention":
            nq, nk, nv = m["heads"] * m["dim"], m["kv_heads"] * m["dim"], m["kv_heads"] * m["vdim"]
            w = mix.proj.weight.float()
            assert torch.equal(w[:nq], t("q")) and torch.equal(w[nq:nq + nk], t("k"))
            assert torch.equal(w[nq + nk:nq + nk + nv], t("v")) and torch.equal(w[nq + nk + nv:], t("g"))
            assert torch.equal(mix.proj.bias.float()[nq:nq + nk], t("k.b")) and not mix.proj.bias[nq + nk + nv:].any()
            assert torch.equal(mix.conv.weight[nq + nk:], t("v.conv")) and mix.conv.weight.dtype == torch.float32
        elif entry["type"] == "mamba2":
            assert torch.equal(mix.in_proj.weight.float(), t("in")) and torch.equal(mix.rec.A_log, t("A_log"))
            assert torch.equal(mix.conv.bias, t("conv.b")) and torch.equal(mix.norm.weight, t("norm"))
        else:
            nq = m["heads"] * m["dim"]
            assert torch.equal(mix.proj.weight.float()[nq:2 * nq], t("k")) and torch.equal(mix.norm.weight, t("norm"))
            assert torch.allclose(mix.rec.decay, torch.tensor(m["decay"]))
    assert torch.equal(model.lm_head.weight.float(), tensors["head"].float())
    assert torch.equal(model.norm.weight, tensors["final.norm"].float())


def test_float32_is_refused_for_16_bit_models():
    from nanovllm.engine.model_runner import _resolve_dtype
    from nanovllm.models.models_map import model_dict
    with pytest.raises(ValueError):
        _resolve_dtype(SimpleNamespace(dtype="bfloat16"), "float32", model_dict["Qwen3ForCausalLM"])
    assert _resolve_dtype(SimpleNamespace(dtype="bfloat16"), "float32", model_dict["Zegopel"]) == torch.float32
    assert _resolve_dtype(SimpleNamespace(dtype="bfloat16"), "auto", model_dict["Zegopel"]) == torch.bfloat16
