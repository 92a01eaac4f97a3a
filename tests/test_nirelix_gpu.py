"""-m gpu: the Nirelix decoder (retention, gated delta rule with per-channel decay, latent attention in a sliding
window, on a residual kept in several streams; clamped gated unit and grouped sigmoid mixture of experts) against
tests/nirelix_oracle.py, a plain float64 restatement.

Every test makes its own small configuration and random weights. Models run in true fp32 (the sharp comparison:
relative error of every row of logits below 2e-4) and in bf16 (the serving precision). The schedules are fed through
LLMEngine.step_given -- the scheduler's block manager, the runner's step and the model's kernels -- so what is
compared is the engine, not a forward function. Where random weights would hide a fault (a window's edge, a key far
back, a block border) the mechanism tests scale one query and key so that one score stands out.
"""
import json
import math
import os
import random

import pytest
import torch

import nirelix_oracle as O

pytestmark = pytest.mark.gpu
F64 = torch.float64


def retention(heads, dim, vdim, dims, base=1000.0, decay=None, mlp=None):
    decay = decay or [0.6 + 0.399 * i / max(1, heads - 1) for i in range(heads)]
    return {"type": "retention", "mlp": mlp,
            "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "decay": decay, "rot": {"dims": dims, "base": base}}}


def delta(heads, kv, dim, vdim, conv, mlp=None):
    return {"type": "channel_delta", "mlp": mlp,
            "mixer": {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "conv": conv}}


def latent(heads, dim, rot, vdim, rank, q_rank, window, scale, base=50.0, mlp=None):
    m = {"heads": heads, "dim": dim, "rot_dim": rot, "vdim": vdim, "kv_rank": rank, "q_rank": q_rank,
         "rot": {"dims": rot, "base": base}, "scale": scale}
    if window:
        m["mask"] = {"size": window}
    return {"type": "latent_attention", "mlp": mlp, "mixer": m}


def dense(ff, limit):
    return {"kind": "dense", "ff": ff, "limit": limit}


def moe(experts, top, ff, count, keep, scale):
    return {"kind": "moe", "expert": {"ff": ff},
            "router": {"experts": experts, "top": top, "groups": {"count": count, "keep": keep}, "scale": scale}}


def config_a():
    """Odd sizes everywhere: three streams, partial rotation, 2 key/value heads under 4 delta heads, key size 72
    (two lanes per state column), a window of 19 tokens over blocks of 16, 6 experts in 3 groups of which 2 stay,
    a layer without feed-forward."""
    return {"architecture": "Nirelix", "vocab": 203, "width": 96, "norm": {"eps": 1e-5}, "streams": 3,
            "layers": [retention(3, 16, 24, 8, mlp=dense(80, 0.7)),
                       delta(4, 2, 24, 20, 3, mlp=moe(6, 3, 40, 3, 2, 2.5)),
                       latent(3, 24, 8, 12, 40, 36, 19, 0.2),
                       delta(2, 2, 72, 16, 2, mlp=dense(56, 1.5)),
                       latent(2, 16, 4, 20, 24, 20, 33, 0.3, base=10000.0, mlp=moe(4, 1, 24, 4, 2, 1.0))]}


def config_b():
    """Values that are 1 or equal: one stream, one key/value head, every expert chosen (no discrete choice: the
    strict bf16 comparison), one group, full rotation, no window entry; width 128 and expert size 64 (the
    tensor-core expert kernels in 16-bit), five taps."""
    return {"architecture": "Nirelix", "vocab": 320, "width": 128, "norm": {"eps": 1e-6}, "streams": 1,
            "layers": [delta(4, 1, 32, 32, 5, mlp=moe(2, 2, 64, 1, 1, 1.5)),
                       retention(2, 64, 32, 64, base=1e6, mlp=dense(128, 1.0)),
                       latent(4, 32, 16, 32, 64, 48, 0, 0.15, mlp=dense(64, 2.0)),
                       retention(4, 32, 48, 16, decay=[0.9, 0.99, 0.999, 1.0])]}


def config_c():
    """No "streams" key at all: a plain residual without stream weights."""
    c = config_b()
    del c["streams"]
    c["layers"] = c["layers"][:3]
    return c


CONFIGS = {"a": config_a, "b": config_b, "c": config_c}
STRICT_BF16 = {"a": False, "b": True, "c": True}
_MODELS = {}


def model_dir(tmp_path_factory, name):
    """(folder with config.json + model.safetensors, config, float64 tensors) of a named test model, made once."""
    if name not in _MODELS:
        from safetensors.torch import save_file
        cfg = CONFIGS[name]()
        tensors = O.random_model(cfg, seed=len(name) + ord(name[0]), ranks=(5, 3) if name == "a" else (8, 16))
        d = tmp_path_factory.mktemp("nirelix_" + name)
        with open(os.path.join(d, "config.json"), "w") as f:
            json.dump(cfg, f)
        save_file({k: v.contiguous() for k, v in tensors.items()}, os.path.join(d, "model.safetensors"))
        _MODELS[name] = (str(d), cfg, O.as_f64(tensors))
    return _MODELS[name]


_ENGINES = {}


def engine(tmp_path_factory, name, dtype, eager=False, blocks=24, block_size=16):
    key = (name, dtype, eager, blocks, block_size)
    if key not in _ENGINES:
        from nanovllm.engine.llm_engine import LLMEngine
        path, cfg, tensors = model_dir(tmp_path_factory, name)
        _ENGINES[key] = LLMEngine(path, dtype=dtype, kvcache_block_size=block_size, num_kvcache_blocks=blocks + 1,
                                  max_num_seqs=4, max_model_len=blocks * block_size,
                                  max_num_batched_tokens=4 * blocks * block_size, return_logits=True,
                                  enforce_eager=eager, chunked_prefill=True)
    return _ENGINES[key], _MODELS[name][1], _MODELS[name][2]


def row_err(got, want):
    """Per row: root mean square of the difference (row means removed) over that of the reference."""
    d = got.to(F64).cpu() - want
    d = d - d.mean(-1, keepdim=True)
    w = want - want.mean(-1, keepdim=True)
    return d.pow(2).mean(-1).sqrt() / w.pow(2).mean(-1).sqrt()


def fp32_noise(cfg, tensors, toks, want):
    """Per row, the error of the oracle itself when it runs in fp32: some prompts drive a norm's input near zero and
    amplify any fp32 rounding; there an fp32 engine is asked to stay within 3 times of that, not below 2e-4."""
    return row_err(O.forward(cfg, {k: v.float() for k, v in tensors.items()}, toks), want)


def close(got, want, dtype, strict=True, noise=None):
    e = row_err(got, want)
    if dtype == "float32":
        limit = torch.full_like(e, 2e-4) if noise is None else torch.maximum(torch.full_like(e, 2e-4), 3 * noise)
        return bool((e < limit).all())
    if strict:
        return float(e.pow(2).mean().sqrt()) < 3e-2 and float(e.max()) < 0.2
    # a model that chooses experts: bf16 rounding may flip a close choice for a token, so a few rows may differ
    return float(e.median()) < 3e-2 and float((e < 0.2).double().mean()) >= 0.9


def tokens_of(cfg, n, seed):
    g = random.Random(seed)
    return [g.randrange(cfg["vocab"]) for _ in range(n)]


def feed(eng, rid, toks, cuts):
    """One request alone, cut at `cuts`; returns logits of every position."""
    outs, lo = [], 0
    for hi in list(cuts) + [len(toks)]:
        if hi <= lo:
            continue
        outs.append(eng.step_given([(rid, toks[lo:hi], list(range(hi - lo)))], [rid] if hi == len(toks) else []))
        lo = hi
    return torch.cat(outs)


CASES = [("a", "float32"), ("a", "bfloat16"), ("b", "float32"), ("b", "bfloat16"), ("c", "float32")]


# ------------------------------------------------------------------ whole prompts, decoding, portions
@pytest.mark.parametrize("name,dtype", CASES)
def test_whole_prompt_and_layers(tmp_path_factory, name, dtype):
    eng, cfg, tensors = engine(tmp_path_factory, name, dtype)
    toks = tokens_of(cfg, 75, 1)
    want, layers = O.forward(cfg, tensors, toks, return_layers=True)
    model = eng.model_runner.model
    model.trace_layers = []
    try:
        got = feed(eng, "w", toks, [])
        seen = [x.cpu() for x in model.trace_layers]
    finally:
        model.trace_layers = None
    assert len(seen) == len(cfg["layers"])
    if dtype == "float32":
        for i, x in enumerate(seen):                  # the sum of the streams after every layer
            assert float((x.to(F64) - layers[i]).abs().max() / layers[i].abs().max()) < 2e-4, i
    assert close(got, want, dtype, STRICT_BF16[name])


@pytest.mark.parametrize("name,dtype", CASES[:4])
@pytest.mark.parametrize("eager", [False, True])
def test_prefill_then_token_by_token(tmp_path_factory, name, dtype, eager):
    """Most of a prompt in one step, the rest one token a step (CUDA-graph decode and eager decode): decoded
    positions cross block borders, leave the windows behind and go well past the convolution tails."""
    eng, cfg, tensors = engine(tmp_path_factory, name, dtype, eager)
    toks = tokens_of(cfg, 70, 2)
    want = O.forward(cfg, tensors, toks)
    for first in (1, 2, 29):
        got = feed(eng, "d", toks, range(first, len(toks)))
        assert close(got, want, dtype, STRICT_BF16[name]), first


@pytest.mark.parametrize("name,dtype", CASES)
def test_portions_of_every_size(tmp_path_factory, name, dtype):
    eng, cfg, tensors = engine(tmp_path_factory, name, dtype)
    toks = tokens_of(cfg, 90, 3)
    want = O.forward(cfg, tensors, toks)
    for size in (2, 3, 7, 16, 19, 33):
        got = feed(eng, "p", toks, range(size, len(toks), size))
        assert close(got, want, dtype, STRICT_BF16[name]), size
    g = random.Random(5)
    cuts, at = [], 0
    while at < len(toks):
        at += g.choice([1, 1, 2, 2, 3, 5, 16, 21])
        cuts.append(at)
    got = feed(eng, "p", toks, [c for c in cuts if c < len(toks)])
    assert close(got, want, dtype, STRICT_BF16[name])


@pytest.mark.parametrize("name,dtype", CASES[:4])
def test_unequal_batches_and_reused_slots(tmp_path_factory, name, dtype):
    """Up to four live requests, portions of some beside single tokens of others, requests that sit out a step;
    every request ends at its own time and later ones take over its blocks and state slot (the pool has 12 blocks,
    the seven requests need 23); each must match its own run alone."""
    pool = 12
    eng, cfg, tensors = engine(tmp_path_factory, name, dtype, blocks=pool)
    g = random.Random(7)
    lens = [37, 90, 5, 64, 51, 33, 18]
    reqs = {f"r{i}": tokens_of(cfg, n, 10 + i) for i, n in enumerate(lens)}
    want = {k: O.forward(cfg, tensors, v) for k, v in reqs.items()}
    noise = {k: fp32_noise(cfg, tensors, v, want[k]) if dtype == "float32" else None for k, v in reqs.items()}
    at = {k: 0 for k in reqs}
    got = {k: [] for k in reqs}
    waiting, live = list(reqs), []
    bm = eng.scheduler.block_manager
    blocks_of = lambda k: -(-len(reqs[k]) // bm.block_size)
    slots, tables = {}, {}
    while waiting or live:
        while waiting and len(live) < 4 and sum(map(blocks_of, live)) + blocks_of(waiting[0]) <= pool:
            live.append(waiting.pop(0))
        entries, end = [], []
        for k in live:
            if at[k] > 0 and g.random() < 0.15:
                continue                                   # left out of this step, goes on later
            n = min(len(reqs[k]) - at[k], g.choice([1, 1, 1, 2, 3, 11, 24]))
            entries.append((k, reqs[k][at[k]:at[k] + n], list(range(n))))
            at[k] += n
            if at[k] == len(reqs[k]):
                end.append(k)
        if not entries:
            continue
        out = eng.step_given(entries, end)
        row = 0
        for k, t, w in entries:
            got[k].append(out[row:row + len(w)])
            row += len(w)
            if k in eng.scheduler.given:
                slots[k] = eng.scheduler.given[k].state_slot
                tables[k] = list(eng.scheduler.given[k].block_table)
        live = [k for k in live if k not in end]
    assert len(set(slots.values())) <= 4 < len(slots)                            # slots were used again
    assert sum(len(t) for t in tables.values()) > pool                           # and so were blocks
    assert len(bm.free_block_ids) == pool and len(bm.free_state_slots) == 4      # everything was given back
    for k in reqs:
        assert close(torch.cat(got[k]), want[k], dtype, STRICT_BF16[name], noise[k]), \
            (k, float(row_err(torch.cat(got[k]), want[k]).max()))


def test_long_decoding(tmp_path_factory):
    """300 tokens one by one after a 3-token prompt in fp32: states and tails are carried 300 times, both windows
    pass over decoded tokens only, attention reads 19 blocks through the table; the logits still match."""
    eng, cfg, tensors = engine(tmp_path_factory, "a", "float32", blocks=20)
    toks = tokens_of(cfg, 303, 4)
    want = O.forward(cfg, tensors, toks)
    got = feed(eng, "l", toks, range(3, len(toks)))
    assert float(row_err(got, want).max()) < 2e-4


def test_greedy_generation_through_the_scheduler(tmp_path_factory):
    """LLM.generate (waiting/running queues, prefill steps, graph decode steps, sampling) in fp32 against the
    oracle's greedy continuation, for three prompts of unequal length at once."""
    from nanovllm import LLM, SamplingParams
    path, cfg, tensors = model_dir(tmp_path_factory, "b")
    llm = LLM(path, dtype="float32", kvcache_block_size=16, num_kvcache_blocks=40, max_num_seqs=4, max_model_len=128,
              max_num_batched_tokens=512)
    prompts = [tokens_of(cfg, n, 20 + n) for n in (9, 30, 17)]
    outs = llm.generate(prompts, SamplingParams(temperature=1.0, max_tokens=10, ignore_eos=True, greedy=True),
                        use_tqdm=False)
    for p, o in zip(prompts, outs):
        seq = list(p)
        for tok in o["token_ids"]:
            logits = O.forward(cfg, tensors, seq)[-1]
            top = torch.topk(logits, 2).values
            if float(top[0] - top[1]) > 1e-3 * float(logits.abs().max()):
                assert tok == int(logits.argmax()), (len(seq), tok)
            seq.append(tok)
    llm.exit()


# ------------------------------------------------------------------ mechanisms alone
def _dev(x, dtype=torch.float32):
    return x.to(dtype).cuda()


def _spans(q_lens, k_lens):
    from nanovllm import ops
    cu_q = torch.tensor([0] + list(torch.tensor(q_lens).cumsum(0)), dtype=torch.int32).cuda()
    cu_k = torch.tensor([0] + list(torch.tensor(k_lens).cumsum(0)), dtype=torch.int32).cuda()
    return ops.StepSpans(cu_q, cu_k, None, max(q_lens))


def _decode_spans(ctx_lens):
    from nanovllm import ops
    return ops.StepSpans(None, None, torch.tensor(ctx_lens, dtype=torch.int32).cuda())


@pytest.mark.parametrize("S,W,kind", [(1, 37, "layer"), (3, 96, "layer"), (8, 40, "layer"), (4, 64, "rms")])
def test_stream_mix_and_norm(S, W, kind):
    """All streams are rewritten from the OLD ones, then read with the next sublayer's weights and normed."""
    from nanovllm import ops
    g = torch.Generator().manual_seed(S * W)
    T = 11
    X = torch.randn(T, S, W, generator=g) * 3
    y = torch.randn(T, W, generator=g)
    mix, out_w, in_w = torch.randn(S, S, generator=g), torch.randn(S, generator=g), torch.randn(S, generator=g)
    w, b = 1 + 0.3 * torch.randn(W, generator=g), torch.randn(W, generator=g)
    eps = 1e-3
    Xn = torch.einsum("st,nsw->ntw", mix.to(F64), X.to(F64)) + out_w.to(F64)[None, :, None] * y.to(F64)[:, None, :]

    def norm(u):
        if kind == "layer":
            return O.layer_norm(u, w.to(F64), b.to(F64), eps)
        return O.rms_unit(u, eps) * (0.5 + w.to(F64))

    xd = _dev(X)
    h, u = ops.stream_mix_norm_(xd, _dev(y), _dev(mix), _dev(out_w), _dev(in_w), _dev(w), _dev(b) if kind == "layer" else None,
                                eps, torch.float32, kind=kind, offset=0.5, sum_out=True)
    want_u = torch.einsum("t,ntw->nw", in_w.to(F64), Xn)
    assert torch.allclose(xd.cpu().to(F64), Xn, atol=1e-5)
    assert torch.allclose(u.cpu().to(F64), want_u, atol=1e-4)
    assert torch.allclose(h.cpu().to(F64), norm(want_u), atol=1e-4)
    # no update, plain sum of the streams (the model's output read)
    h2 = ops.stream_mix_norm_(xd, None, None, None, None, _dev(w), _dev(b) if kind == "layer" else None, eps,
                              torch.float32, kind=kind, offset=0.5)
    assert torch.allclose(h2.cpu().to(F64), norm(Xn.sum(1)), atol=1e-4)


@pytest.mark.parametrize("interleaved", [False, True])
def test_rotary_on_part_of_a_head(interleaved):
    """Partial rotation at positions up to 10^5 (angles in fp64), a scale for the second half of the heads only,
    strided input, output into a wider head."""
    from nanovllm import ops
    g = torch.Generator().manual_seed(3)
    T, H, width, dims, base = 9, 4, 24, 10, 777.0
    pos = torch.tensor([0, 1, 2, 17, 95, 1000, 4097, 65536, 100001])
    big = torch.randn(T, H * width + 5, generator=g)
    x = big[:, 3:3 + H * width].view(T, H, width)
    want = O.rotate(x.to(F64), pos, dims, base, interleaved)
    want[:, 2:] *= 0.25
    xd = _dev(big)[:, 3:3 + H * width].unflatten(1, (H, width))
    got = ops.rotary_heads(xd, pos.cuda(), H, width, dims, base, interleaved, out_f32=True, split=2, scale_hi=0.25)
    assert torch.allclose(got.cpu().to(F64), want, atol=2e-6)
    wide = torch.zeros(T, H, width + 7, device="cuda")
    ops.rotary_heads(xd, pos.cuda(), H, width, dims, base, interleaved, out=wide[:, :, 7:], split=2, scale_hi=0.25)
    assert torch.allclose(wide[:, :, 7:].cpu().to(F64), want, atol=2e-6) and float(wide[:, :, :7].abs().max()) == 0
    hb = ops.rotary_heads(xd.bfloat16(), pos.cuda(), H, width, dims, base, interleaved, out_f32=True)
    assert torch.allclose(hb.cpu().to(F64), O.rotate(x.bfloat16().to(F64), pos, dims, base, interleaved), atol=2e-6)


@pytest.mark.parametrize("inter", [13, 64])
def test_clamped_gated_unit(inter):
    from nanovllm import ops
    g = torch.Generator().manual_seed(inter)
    x = torch.randn(7, 2 * inter, generator=g) * 3
    x[0, :4] = torch.tensor([9.0, -9.0, 0.7, -0.7])
    x[0, inter:inter + 4] = torch.tensor([-9.0, 9.0, 0.7, -0.7])
    limit, alpha = 0.7, 1.702
    gate, up = x[:, :inter].to(F64).clamp(max=limit), x[:, inter:].to(F64).clamp(-limit, limit)
    want = gate * torch.sigmoid(alpha * gate) * (up + 1)
    got = ops.glu_clamped(_dev(x), alpha, limit)
    assert torch.allclose(got.cpu().to(F64), want, atol=1e-6)


@pytest.mark.parametrize("E,top,count,keep", [(6, 3, 3, 2), (12, 2, 2, 1), (8, 1, 1, 1), (8, 3, 8, 5), (64, 8, 8, 4),
                                              (5, 5, 1, 1), (9, 2, 3, 3)])
def test_grouped_sigmoid_router(E, top, count, keep):
    """Choice scores include the correction (negative ones too: a group outside the kept ones counts as minus
    infinity, not zero), the weights do not; groups of one expert score that expert alone."""
    from nanovllm import ops
    g = torch.Generator().manual_seed(E * top)
    T = 200
    z = torch.randn(T, E, generator=g) * 2
    corr = torch.randn(E, generator=g) - 1.5
    r = {"experts": E, "top": top, "groups": {"count": count, "keep": keep}, "scale": 1.7}
    idx, w = O.route(z.to(F64), corr.to(F64), r)
    ids, wg = ops.moe_route_grouped(_dev(z), _dev(corr), top, count, keep, 1.7)
    ids, wg = ids.cpu().long(), wg.cpu().to(F64)
    order_w, order_g = idx.argsort(-1), ids.argsort(-1)
    assert torch.equal(idx.gather(1, order_w), ids.gather(1, order_g))
    assert torch.allclose(w.gather(1, order_w), wg.gather(1, order_g), atol=1e-6)


def _moe_case(W, ff, E, top, count, keep, dtype, fast, seed, tokens=150):
    from nanovllm.layers.moe import GroupedSigmoidMoe
    cfg = {"architecture": "Nirelix", "vocab": 8, "width": W, "norm": {"eps": 1e-6},
           "layers": [dict(delta(1, 1, 8, 8, 2), mlp=moe(E, top, ff, count, keep, 1.3))]}
    t = O.as_f64(O.random_model(cfg, seed))
    P = O.sub(t, "l0.mlp.")
    prev = torch.get_default_dtype()
    torch.set_default_dtype(dtype)
    try:
        with torch.device("cuda"):
            m = GroupedSigmoidMoe(W, ff, E, top, count, keep, 1.3)
    finally:
        torch.set_default_dtype(prev)
    m.fast = fast
    m.router.data.copy_(P["router"])
    m.correction.data.copy_(P["correction"])
    for e in range(E):
        m.w13.data[e, :ff].copy_(P[f"e{e}.gate"])
        m.w13.data[e, ff:].copy_(P[f"e{e}.up"])
        m.w2.data[e].copy_(P[f"e{e}.down"])
    x = torch.randn(tokens, W, generator=torch.Generator().manual_seed(seed)).to(dtype)
    want = O.moe_ff(x.to(F64), P, cfg["layers"][0]["mlp"])
    with torch.no_grad():
        got = m(x.cuda())
    return (got.cpu().to(F64) - want).norm(dim=-1) / want.norm(dim=-1)


def test_mixture_of_experts_any_size_fp32():
    e = _moe_case(40, 24, 6, 3, 3, 2, torch.float32, True, 1)
    assert float(e.max()) < 1e-5
    e = _moe_case(128, 64, 8, 2, 2, 1, torch.float32, True, 2)
    assert float(e.max()) < 1e-5


@pytest.mark.parametrize("fast,tokens", [(True, 150), (True, 1000), (False, 150)])
def test_mixture_of_experts_bf16_both_paths(fast, tokens):
    """Width 128 and expert size 64 fit the tensor-core expert kernels (fast: the weight-streaming form for few rows
    per expert, the grouped tcgen05 form for many) and run on the generic ones as well; a few tokens may choose
    differently than the float64 oracle after the input's rounding."""
    e = _moe_case(128, 64, 8, 2, 2, 1, torch.bfloat16, fast, 3, tokens)
    assert float(e.median()) < 1e-2 and float((e < 3e-2).double().mean()) > 0.9


def test_delta_prep_formulas():
    """Unit vectors with the epsilon inside the root (a zero head stays zero), softplus in its linear range, decay
    laid out heads x key channels."""
    from nanovllm import ops
    g = torch.Generator().manual_seed(9)
    T, H, G, d = 6, 4, 2, 12
    qk = torch.randn(T, 2 * G * d, generator=g)
    qk[0, :d] = 0
    a = torch.randn(T, H * d, generator=g) * 3
    a[1, :5] = torch.tensor([40.0, -40.0, 25.0, 0.0, 88.0])
    b = torch.randn(T, H, generator=g)
    dt_bias, a_log = torch.randn(H * d, generator=g), torch.randn(H, generator=g)
    qk32, dec, beta = ops.delta_prep(_dev(qk), _dev(a), _dev(b), _dev(dt_bias), _dev(a_log), H, G, d, 1e-6, d ** -0.5)
    x = qk.to(F64).view(T, 2 * G, d)
    unit = x / torch.sqrt(x.pow(2).sum(-1, keepdim=True) + 1e-6)
    unit[:, :G] *= d ** -0.5
    assert torch.allclose(qk32.cpu().to(F64), unit.reshape(T, -1), atol=1e-6)
    want = torch.exp(-torch.exp(a_log.to(F64))[None, :, None] * O.softplus((a + dt_bias).to(F64).view(T, H, d)))
    assert torch.allclose(dec.cpu().to(F64), want.reshape(T, -1), atol=1e-6)
    assert torch.allclose(beta.cpu().to(F64), torch.sigmoid(b.to(F64)), atol=1e-6)


@pytest.mark.parametrize("H,G,d,dv", [(4, 2, 24, 20), (2, 2, 72, 16), (1, 1, 130, 40), (2, 1, 16, 130), (3, 3, 64, 64)])
@pytest.mark.parametrize("vdtype", [torch.float32, torch.bfloat16])
def test_delta_rule_in_portions(H, G, d, dv, vdtype):
    """Two sequences in slots 3 and 1 fed in portions of 1..40 tokens, then single tokens as decode rows: equals the
    recurrence over each whole sequence; a slot that held another state is ignored at position 0."""
    from nanovllm import ops
    g = torch.Generator().manual_seed(H * d + dv)
    lens = [61, 23]
    seqs = []
    for n in lens:
        q = torch.randn(n, G * d, generator=g) * d ** -0.5
        k = torch.nn.functional.normalize(torch.randn(n, G, d, generator=g), dim=-1).reshape(n, G * d)
        v = torch.randn(n, H * dv, generator=g).to(vdtype).float()
        gate = torch.rand(n, H * d, generator=g) * 0.3 + 0.7
        beta = torch.rand(n, H, generator=g)
        seqs.append((q, k, v, gate, beta))
    want = []
    rep = H // G
    for (q, k, v, gate, beta), n in zip(seqs, lens):
        want.append(O.delta_recurrence(q.to(F64).view(n, G, d).repeat_interleave(rep, 1),
                                       k.to(F64).view(n, G, d).repeat_interleave(rep, 1), v.to(F64).view(n, H, dv),
                                       gate.to(F64).view(n, H, d), beta.to(F64)).reshape(n, H * dv))
    state = torch.full((5, H, d, dv), 7.0, device="cuda")
    slots = torch.tensor([3, 1], dtype=torch.int32).cuda()
    got, at = [[], []], [0, 0]
    portions = [[1, 2], [2, 1], [40, 3], [3, 16]] + [[1, 1]] * 3 + [[12, 0]]
    for portion in portions:
        q = [min(p, lens[i] - at[i]) for i, p in enumerate(portion)]
        live = [i for i in range(2) if q[i] > 0]
        if portion == [1, 1]:
            sp = _decode_spans([at[i] + 1 for i in live])
        else:
            sp = _spans([q[i] for i in live], [at[i] + q[i] for i in live])
        cat = lambda j, dt=torch.float32: torch.cat([seqs[i][j][at[i]:at[i] + q[i]] for i in live]).to(dt).cuda()
        out = ops.delta_rule(cat(0), cat(1), cat(2, vdtype), cat(3), cat(4), sp, H, G, d, dv, state,
                             slots[live].contiguous())
        row = 0
        for i in live:
            got[i].append(out[row:row + q[i]].cpu())
            row += q[i]
            at[i] += q[i]
    for i in range(2):
        o = torch.cat(got[i]).to(F64)
        assert o.shape[0] == at[i]
        assert float((o - want[i][:at[i]]).abs().max() / want[i].abs().max()) < 2e-5, i


def test_delta_rule_far_token_and_overwrite():
    """A value written under key e0 500 tokens back is read almost undamped with decays of 0.9999 and is gone with
    0.9; writing the same key again with beta = 1 replaces the old value."""
    from nanovllm import ops
    H, d, dv, n = 1, 32, 8, 502
    for decay, survives in ((0.9999, True), (0.9, False)):
        k = torch.zeros(n, d)
        k[0, 0] = 1.0
        k[1:, 1:] = torch.nn.functional.normalize(torch.randn(n - 1, d - 1, generator=torch.Generator().manual_seed(1)), dim=-1)
        q = torch.zeros(n, d)
        q[-1, 0] = 1.0
        v = torch.randn(n, dv, generator=torch.Generator().manual_seed(2))
        gate = torch.full((n, d), decay)
        beta = torch.ones(n, 1)
        state = torch.zeros(2, H, d, dv, device="cuda")
        slots = torch.tensor([1], dtype=torch.int32).cuda()
        out = ops.delta_rule(_dev(q[:400]), _dev(k[:400]), _dev(v[:400]), _dev(gate[:400]), _dev(beta[:400]),
                             _spans([400], [400]), H, H, d, dv, state, slots)
        for t in range(400, n):                       # the rest one token a step
            out = ops.delta_rule(_dev(q[t:t + 1]), _dev(k[t:t + 1]), _dev(v[t:t + 1]), _dev(gate[t:t + 1]),
                                 _dev(beta[t:t + 1]), _decode_spans([t + 1]), H, H, d, dv, state, slots)
        want = v[0].to(F64) * decay ** (n - 1)
        got = out[0].cpu().to(F64)
        if survives:
            assert torch.allclose(got, want, atol=1e-4) and float(want.abs().max()) > 0.5
        else:
            assert float(got.abs().max()) < 1e-12
    k2 = torch.zeros(2, d)
    k2[:, 0] = 1.0
    v2 = torch.randn(2, dv, generator=torch.Generator().manual_seed(3))
    q2 = k2.clone()
    out = ops.delta_rule(_dev(q2), _dev(k2), _dev(v2), torch.ones(2, d, device="cuda"), torch.ones(2, 1, device="cuda"),
                         _spans([2], [2]), H, H, d, dv)
    assert torch.allclose(out.cpu(), v2, atol=1e-6)


@pytest.mark.parametrize("vdtype", [torch.float32, torch.bfloat16])
def test_retention_fp32_queries_beside_projected_values(vdtype):
    """The constant-decay recurrence with q, k in fp32 (rotated upstream) and v as projected; 45-token portions, then
    single tokens; a token 500 steps back survives a decay of 0.999 and is gone at 0.5."""
    from nanovllm import ops
    H, d, dv, n = 2, 20, 12, 520
    g = torch.Generator().manual_seed(4)
    q, k = torch.randn(n, H * d, generator=g), torch.randn(n, H * d, generator=g) * 0.05
    v = torch.randn(n, H * dv, generator=g).to(vdtype).float()
    k[0] = 0
    k[0, 0], k[0, d] = 30.0, 30.0                        # one loud write at position 0, both heads
    q[-1] = 0
    q[-1, 0], q[-1, d] = 1.0, 1.0
    decay = [0.999, 0.5]
    want = O.retention_recurrence(q.to(F64).view(n, H, d), k.to(F64).view(n, H, d), v.to(F64).view(n, H, dv), decay)
    state = torch.full((3, H, d, dv), 5.0, device="cuda")
    slots = torch.tensor([2], dtype=torch.int32).cuda()
    dec = torch.tensor(decay).cuda()
    outs, at = [], 0
    while at < n:
        step = 45 if at < 450 else 1
        step = min(step, n - at)
        sp = _spans([step], [at + step]) if step > 1 else _decode_spans([at + 1])
        outs.append(ops.linear_recurrence(_dev(q[at:at + step]), _dev(k[at:at + step]), _dev(v[at:at + step], vdtype), sp,
                                          H, H, d, dv, state, slots, decay=dec).cpu())
        at += step
    got = torch.cat(outs).to(F64).view(n, H, dv)
    assert float((got - want).abs().max() / want.abs().max()) < 2e-5
    far = 30.0 * v[0].to(F64).view(H, dv)
    assert float((got[-1, 0] - want[-1, 0]).abs().max()) < 1e-3 and float(want[-1, 0].abs().max()) > 0.3 * float(far[0].abs().max()) * 0.999 ** n
    assert float(got[-1, 1].abs().max()) < 1.0            # decay 0.5: the loud write is gone, only recent tokens remain


def _latent_case(n, window, star, dtype, dim=40, rank=24, H=3, seed=0):
    """Keys of one latent head: random and quiet, except key `star`, which every query's first head is scaled to
    find. Returns (q [n, H, dim], rows [n, dim], expected [n, H, rank]) with values = the first `rank` columns."""
    g = torch.Generator().manual_seed(seed)
    rows = (torch.randn(n, dim, generator=g) * 0.3).to(dtype).to(F64)
    q = (torch.randn(n, H, dim, generator=g) * 0.3).to(dtype).to(F64)
    if star is not None:
        rows[star] = (rows[star] * 10).to(dtype).to(F64)
        q[:, 0] = (rows[star] * 2)[None].to(dtype).to(F64)
    want = torch.zeros(n, H, rank, dtype=F64)
    for i in range(n):
        lo = max(0, i - window + 1) if window else 0
        for h in range(H):
            p = torch.softmax(rows[lo:i + 1] @ q[i, h] * 0.5, 0)
            want[i, h] = p @ rows[lo:i + 1, :rank]
    return q, rows, want


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_window_edges_in_prompts_and_decoding(dtype):
    """A loud key at position 37 with a window of 19 over blocks of 16 (shuffled table): the query at 37 + 18 still
    finds it, the one at 37 + 19 does not; as a prompt portion that starts inside the window and as single decoded
    tokens; values are the first columns of the cached rows."""
    from nanovllm import ops
    n, window, star, rank, dim, H = 80, 19, 37, 24, 40, 3
    q, rows, want = _latent_case(n, window, star, dtype)
    inside, outside = want[star + window - 1, 0], want[star + window, 0]
    assert float((inside - rows[star, :rank]).abs().max()) < 1e-2 < float((outside - rows[star, :rank]).abs().max())
    bs, nb = 16, 9
    table = torch.tensor([[7, 2, 5, 0, 3, 8]], dtype=torch.int32).cuda()
    cache = torch.zeros(nb, bs, dim, dtype=dtype, device="cuda")
    for j in range(n):
        cache[int(table[0, j // bs]), j % bs] = rows[j].to(dtype)
    tol = 1e-5 if dtype == torch.float32 else 2e-2
    cut = star + 10
    out = ops.attn_generic(_dev(q[:cut], dtype), cache, None, _spans([cut], [cut]), 0.5, 1, rank, block_tables=table,
                           window=window)
    assert float((out.cpu().to(F64).view(cut, H, rank) - want[:cut]).abs().max()) < tol
    out = ops.attn_generic(_dev(q[cut:], dtype), cache, None, _spans([n - cut], [n]), 0.5, 1, rank, block_tables=table,
                           window=window)                # a portion that starts inside the loud key's window
    assert float((out.cpu().to(F64).view(n - cut, H, rank) - want[cut:]).abs().max()) < tol
    for i in (0, 1, 15, 16, 17, star + window - 2, star + window - 1, star + window, star + window + 1, n - 1):
        out = ops.attn_generic(_dev(q[i:i + 1], dtype), cache, None, _decode_spans([i + 1]), 0.5, 1, rank,
                               block_tables=table, window=window)
        assert float((out.cpu().to(F64).view(H, rank) - want[i]).abs().max()) < tol, i
    # packed keys (no cache bound), two sequences of unequal length in one launch
    q2, rows2, want2 = _latent_case(30, window, 5, dtype, seed=1)
    out = ops.attn_generic(_dev(torch.cat([q, q2]), dtype), _dev(torch.cat([rows, rows2]), dtype).unsqueeze(1), None,
                           _spans([n, 30], [n, 30]), 0.5, 1, rank, window=window)
    assert float((out.cpu().to(F64).view(n + 30, H, rank) - torch.cat([want, want2])).abs().max()) < tol


def test_far_key_without_a_window():
    """Key 3 among 700, no window, key size 576 and value size 512 (the sizes of a large latent)."""
    from nanovllm import ops
    n, rank, dim, H = 700, 512, 576, 2
    q, rows, want = _latent_case(n, 0, 3, torch.float32, dim=dim, rank=rank, H=H, seed=2)
    out = ops.attn_generic(_dev(q[-40:]), _dev(rows).unsqueeze(1), None, _spans([40], [n]), 0.5, 1, rank)
    assert float((out.cpu().to(F64).view(40, H, rank) - want[-40:]).abs().max()) < 1e-4
    assert float((want[-1, 0] - rows[3, :rank]).abs().max()) < 1e-2


def test_window_with_separate_values_and_grouped_heads():
    """The same window in the general form: 4 query heads on 2 key/value heads, values in their own tensor."""
    from nanovllm import ops
    g = torch.Generator().manual_seed(6)
    n, H, G, d, dv, window = 50, 4, 2, 12, 20, 7
    q, k, v = torch.randn(n, H, d, generator=g), torch.randn(n, G, d, generator=g), torch.randn(n, G, dv, generator=g)
    k[20] *= 8
    want = torch.zeros(n, H, dv, dtype=F64)
    for i in range(n):
        lo = max(0, i - window + 1)
        for h in range(H):
            p = torch.softmax(k[lo:i + 1, h // 2].to(F64) @ q[i, h].to(F64) * 0.4, 0)
            want[i, h] = p @ v[lo:i + 1, h // 2].to(F64)
    out = ops.attn_generic(_dev(q), _dev(k), _dev(v), _spans([n], [n]), 0.4, G, dv, window=window)
    assert float((out.cpu().to(F64).view(n, H, dv) - want).abs().max()) < 1e-5


def test_latent_rows_norms_rotation_and_cache_write():
    from nanovllm import ops
    g = torch.Generator().manual_seed(8)
    T, q_rank, rank, rot, eps, base = 7, 20, 24, 6, 1e-5, 50.0
    big = torch.randn(T, 64, generator=g)
    dq, dkv = big[:, :q_rank], big[:, 24:24 + rank + rot]
    wq, wc = 1 + 0.2 * torch.randn(q_rank, generator=g), 1 + 0.2 * torch.randn(rank, generator=g)
    pos = torch.tensor([0, 1, 2, 63, 64, 1000, 50000])
    bd = _dev(big)
    for pairs in (False, True):
        cache = torch.zeros(4, 16, rank + rot, device="cuda")
        flat = torch.tensor([5, 17, 16, 63, 0, 31, 40], dtype=torch.int32)
        slots = torch.stack([flat // 16, flat % 16], 1).contiguous() if pairs else flat
        cq, kc = ops.latent_kv_prep(bd[:, :q_rank], bd[:, 24:24 + rank + rot], _dev(wq), _dev(wc), pos.cuda(), rank, rot,
                                    rot, base, True, eps, cache=cache, slots=slots.cuda())
        assert torch.allclose(cq.cpu().to(F64), O.rms_unit(dq.to(F64), eps) * wq.to(F64), atol=1e-5)
        want = torch.cat([O.rms_unit(dkv[:, :rank].to(F64), eps) * wc.to(F64),
                          O.rotate(dkv[:, None, rank:].to(F64), pos, rot, base, True)[:, 0]], 1)
        assert torch.allclose(kc.cpu().to(F64), want, atol=1e-5)
        assert torch.allclose(cache.view(64, -1)[flat.long()].cpu().to(F64), want, atol=1e-5)


@pytest.mark.parametrize("own", [True, False])
def test_latent_prompts_on_library_products(own):
    """Prompt portions of a 16-bit model run as library products around the masked softmax kernel: a 150-token
    portion that continues 60 cached tokens (three query chunks of 64, key ranges that start inside the window), a
    second whole sequence, and a short portion beside them, over a shuffled block table; same loud key at the
    window's edge as in the kernel's own test. `own`: the scores on the tcgen05 GEMM with fp32 output (key ranges of
    128 rows, rows padded from 40 to 64 columns) or on the library's mixed-precision product."""
    from nanovllm import ops
    from nanovllm.layers.seq_mixers import LatentAttention
    from nanovllm.utils.context import reset_context, set_context
    dtype, window, rank, dim, H, bs = torch.bfloat16, 19, 24, 40, 3, 16
    lens, starts = [210, 100, 30], [60, 0, 21]                # tokens in all, tokens already cached
    stars = [97, 50, 3]
    cases = [_latent_case(n, window, st, dtype, seed=5 + i) for i, (n, st) in enumerate(zip(lens, stars))]
    attn = LatentAttention(H, dim - rank - 4, 4 + 0, 8, rank, 0.5, window=window)      # sizes only matter as rank + rot = 40
    attn.rot = dim - rank
    attn.PRODUCT_CHUNK = 64
    attn.OWN_SCORE_PRODUCT = own
    nb = sum(-(-n // bs) for n in lens)
    order = list(range(nb))
    random.Random(3).shuffle(order)
    attn.k_cache = torch.zeros(nb + 1, bs, dim, dtype=dtype, device="cuda")
    tables, at = [], 0
    for (q, rows, want), n in zip(cases, lens):
        blocks = order[at:at + -(-n // bs)]
        at += len(blocks)
        tables.append(blocks + [-1] * (14 - len(blocks)))
        for j in range(n):
            attn.k_cache[blocks[j // bs], j % bs] = rows[j].to(dtype)
    q_lens = [n - s for n, s in zip(lens, starts)]
    cu_q = [0] + list(torch.tensor(q_lens).cumsum(0).tolist())
    cu_k = [0] + list(torch.tensor(lens).cumsum(0).tolist())
    dev_i32 = lambda x: torch.tensor(x, dtype=torch.int32).cuda()
    set_context(True, cu_seqlens_q=dev_i32(cu_q), cu_seqlens_k=dev_i32(cu_k), max_seqlen_q=max(q_lens),
                max_seqlen_k=max(lens), block_tables=dev_i32(tables), block_size=bs,
                host_spans=[(cu_q[i], q_lens[i], lens[i]) for i in range(3)])
    try:
        from nanovllm.utils.context import get_context
        qx = torch.cat([c[0][s:] for c, s in zip(cases, starts)]).to(dtype).cuda()
        got = attn._prefill_by_products(qx, None, get_context(), True).cpu().to(F64).view(-1, H, rank)
    finally:
        reset_context()
    want = torch.cat([c[2][s:] for c, s in zip(cases, starts)])
    assert float((got - want).abs().max()) < 2e-2
    edge = stars[0] + window - 1 - starts[0]                  # row of the last query that still sees the loud key
    assert float((got[edge, 0] - cases[0][1][stars[0], :rank]).abs().max()) < 3e-2
    assert float((got[edge + 1, 0] - cases[0][1][stars[0], :rank]).abs().max()) > 0.3


@pytest.mark.parametrize("window", [19, 200])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_latent_decode_rows_inside_a_window(dtype, window):
    """Decode steps gather each sequence's last `window` rows: sequences shorter than the window, exactly at it, with
    the loud key just inside and just outside, and a padded row (0 keys) in one launch; a window wider than what a
    block table can hold (200 > 5 blocks of 16) gathers the table's capacity."""
    from nanovllm.layers.seq_mixers import LatentAttention
    from nanovllm.utils.context import get_context, reset_context, set_context
    rank, dim, H, bs, star = 24, 40, 3, 16, 37
    q, rows, want = _latent_case(80, window, star, dtype)
    attn = LatentAttention(H, 12, 16, 8, rank, 0.5, window=window)
    table = [7, 2, 5, 0, 3]
    attn.k_cache = torch.zeros(9, bs, dim, dtype=dtype, device="cuda")
    for j in range(80):
        attn.k_cache[table[j // bs], j % bs] = rows[j].to(dtype)
    at = [4, 18, 19, star + 18, star + 19, 79]                                      # positions of the decoded tokens
    ctx_lens = [p + 1 for p in at] + [0]
    qx = torch.cat([q[at], torch.zeros(1, H, dim, dtype=F64)]).to(dtype).cuda()
    tables = torch.tensor([table] * 6 + [[-1] * 5], dtype=torch.int32).cuda()
    set_context(False, context_lens=torch.tensor(ctx_lens, dtype=torch.int32).cuda(), block_tables=tables, block_size=bs)
    try:
        got = attn._decode_window_by_products(qx, get_context()).cpu().to(F64).view(-1, H, rank)
    finally:
        reset_context()
    assert float((got[:6] - want[at]).abs().max()) < (1e-5 if dtype == torch.float32 else 2e-2)
    assert float(got[6].abs().max()) == 0.0
    if window == 19:
        assert float((got[3, 0] - rows[star, :rank]).abs().max()) < 3e-2 < float((got[4, 0] - rows[star, :rank]).abs().max())


@pytest.mark.parametrize("act", ["sigmoid", "silu"])
def test_norm_per_head_and_gate(act):
    """One RMS norm per head (a warp per head), a weight shared by the heads, then the gate."""
    from nanovllm import ops
    g = torch.Generator().manual_seed(11)
    rows, H, dv, eps = 9, 4, 24, 1e-4
    y, gate = torch.randn(rows, H * dv, generator=g) * 3, torch.randn(rows, H * dv + 8, generator=g)
    w = 1 + 0.2 * torch.randn(dv, generator=g)
    gv = gate[:, 8:].to(F64)
    want = (O.rms_unit(y.to(F64).view(rows, H, dv), eps) * w.to(F64)).reshape(rows, -1) * \
        (torch.sigmoid(gv) if act == "sigmoid" else O.silu(gv))
    got = ops.gated_norm(_dev(y), _dev(gate)[:, 8:], _dev(w.repeat(H)), eps, groups=H, gate_first=False, gate_act=act)
    assert torch.allclose(got.cpu().to(F64), want, atol=1e-5)
