"""-m gpu: the Zegopel hybrid decoder (softmax attention with a short convolution and a query temperature,
lightning attention, Mamba-2) against tests/zegopel_oracle.py, a plain float64 restatement.

Every test makes its own small configuration and random weights. Models run in true fp32 (the sharp
comparison: relative error of every row of logits below 2e-4) and in bf16 (the serving precision: below 3e-2
over all rows together and below 0.2 in the worst row -- single rows of a random model amplify bf16 rounding).
The schedules are fed through LLMEngine.step_given -- the scheduler's block manager, the runner's step and the
model's kernels -- so what is compared is the engine, not a forward function.
"""
import json
import os
import random

import pytest
import torch

import zegopel_oracle as O

pytestmark = pytest.mark.gpu
F64 = torch.float64


def attention(heads, kv, dim, vdim, conv, every, coef=0.4, scale=0.3, ff=None):
    return {"type": "attention", "mlp": {"kind": "dense", "ff": ff} if ff else None,
            "mixer": {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "conv": conv, "scale": scale,
                      "q_temp": {"coef": coef, "every": every}}}


def lightning(heads, dim, vdim, decay=None, ff=None):
    decay = decay or [0.5 + 0.499 * i / max(1, heads - 1) for i in range(heads)]
    return {"type": "lightning", "mlp": {"kind": "dense", "ff": ff} if ff else None,
            "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "decay": decay}}


def mamba2(heads, vdim, state, groups, norm_groups, conv, ff=None):
    return {"type": "mamba2", "mlp": {"kind": "dense", "ff": ff} if ff else None,
            "mixer": {"heads": heads, "vdim": vdim, "state": state, "groups": groups, "norm_groups": norm_groups,
                      "conv": conv}}


def config_a():
    """Odd sizes everywhere: key size != value size, 2 kv heads, taps 4 and 2, a feed-forward after a recurrent
    layer and none after the attention layer, norm groups != groups."""
    return {"architecture": "Zegopel", "vocab": 203, "width": 96, "norm": {"eps": 1e-5},
            "layers": [lightning(3, 16, 24, ff=80), attention(6, 2, 24, 40, 4, 8),
                       mamba2(4, 12, 20, 2, 4, 2, ff=64), attention(2, 2, 48, 16, 2, 5, coef=0.7, scale=0.11)]}


def config_b():
    """Head size 64 = value size (the tcgen05 / paged-decode kernels in 16-bit), one mamba group, one tap
    more than the other configuration, a temperature period larger than the prompts."""
    return {"architecture": "Zegopel", "vocab": 320, "width": 128, "norm": {"eps": 1e-6},
            "layers": [attention(4, 2, 64, 64, 3, 1000, ff=192), mamba2(6, 32, 16, 1, 1, 5),
                       lightning(2, 40, 72), attention(8, 1, 64, 64, 2, 16, ff=96)]}


_MODELS = {}


def model_dir(tmp_path_factory, name):
    """(folder with config.json + model.safetensors, config, tensors) of a named test model, made once."""
    if name not in _MODELS:
        from safetensors.torch import save_file
        cfg = {"a": config_a, "b": config_b}[name]()
        tensors = O.random_model(cfg, seed=len(name) + ord(name[0]))
        d = tmp_path_factory.mktemp("zegopel_" + name)
        with open(os.path.join(d, "config.json"), "w") as f:
            json.dump(cfg, f)
        save_file({k: v.contiguous() for k, v in tensors.items()}, os.path.join(d, "model.safetensors"))
        _MODELS[name] = (str(d), cfg, tensors)
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


def rel_err(got, want):
    """Root mean square of the difference (row means removed) over that of the reference, worst row."""
    d = got.to(F64) - want
    d = d - d.mean(-1, keepdim=True)
    w = want - want.mean(-1, keepdim=True)
    return float((d.pow(2).mean(-1).sqrt() / w.pow(2).mean(-1).sqrt()).max())


LIMIT = {"float32": 2e-4, "bfloat16": 5e-2}


def pooled_err(got, want):
    d = got.to(F64) - want
    d = d - d.mean(-1, keepdim=True)
    w = want - want.mean(-1, keepdim=True)
    return float(d.pow(2).mean().sqrt() / w.pow(2).mean().sqrt())


def close(got, want, dtype):
    if dtype == "float32":
        return rel_err(got, want) < 2e-4
    return pooled_err(got, want) < 3e-2 and rel_err(got, want) < 0.2


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


# ------------------------------------------------------------------ whole prompts, decoding, portions
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["a", "b"])
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
    for i, x in enumerate(seen):                      # the residual stream after every layer
        assert float((x.to(F64) - layers[i]).abs().max() / layers[i].abs().max()) < LIMIT[dtype], i
    assert close(got, want, dtype)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["a", "b"])
@pytest.mark.parametrize("eager", [False, True])
def test_prefill_then_token_by_token(tmp_path_factory, name, dtype, eager):
    """Most of a prompt in one step, the rest one token a step (CUDA-graph decode and eager decode): positions
    cross a block border, the temperature's period, and go well past the convolution tails."""
    eng, cfg, tensors = engine(tmp_path_factory, name, dtype, eager)
    toks = tokens_of(cfg, 70, 2)
    want = O.forward(cfg, tensors, toks)
    for first in (1, 2, 29):
        got = feed(eng, "d", toks, range(first, len(toks)))
        assert close(got, want, dtype), first


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["a", "b"])
def test_portions_of_every_size(tmp_path_factory, name, dtype):
    eng, cfg, tensors = engine(tmp_path_factory, name, dtype)
    toks = tokens_of(cfg, 90, 3)
    want = O.forward(cfg, tensors, toks)
    for size in (2, 3, 7, 16, 17, 33):
        got = feed(eng, "p", toks, range(size, len(toks), size))
        assert close(got, want, dtype), size
    g = random.Random(5)
    cuts, at = [], 0
    while at < len(toks):
        at += g.choice([1, 1, 2, 2, 3, 5, 16, 21])
        cuts.append(at)
    got = feed(eng, "p", toks, [c for c in cuts if c < len(toks)])
    assert close(got, want, dtype)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["a", "b"])
def test_unequal_batches_and_reused_slots(tmp_path_factory, name, dtype):
    """Up to four live requests, portions of some beside single tokens of others, requests that sit out a
    step; every request ends at its own time and later ones take over its blocks and state slot (the pool has
    12 blocks, the seven requests need 23); each must match its own run alone."""
    pool = 12
    eng, cfg, tensors = engine(tmp_path_factory, name, dtype, blocks=pool)
    g = random.Random(7)
    lens = [37, 90, 5, 64, 51, 33, 18]
    reqs = {f"r{i}": tokens_of(cfg, n, 10 + i) for i, n in enumerate(lens)}
    want = {k: O.forward(cfg, tensors, v) for k, v in reqs.items()}
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
        for k, _, _ in entries:                            # what the request holds when it has all its tokens
            if k in end and k in eng.scheduler.given:
                tables[k] = list(eng.scheduler.given[k].block_table)
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
        assert close(torch.cat(got[k]), want[k], dtype), (k, rel_err(torch.cat(got[k]), want[k]))


def test_long_decoding_and_far_tokens(tmp_path_factory):
    """600 tokens one by one after a 3-token prompt in fp32: the recurrent states and tails are carried 600 times,
    attention reads 38 blocks through the table; the logits at the end still match."""
    eng, cfg, tensors = engine(tmp_path_factory, "a", "float32", blocks=40)
    toks = tokens_of(cfg, 603, 4)
    want = O.forward(cfg, tensors, toks)
    got = feed(eng, "l", toks, range(3, len(toks)))
    assert rel_err(got, want) < LIMIT["float32"]
    assert rel_err(got[-50:], want[-50:]) < LIMIT["float32"]


def test_greedy_generation_through_the_scheduler(tmp_path_factory):
    """LLM.generate (waiting/running queues, prefill steps, graph decode steps, sampling) in fp32 against the
    oracle's greedy continuation, for three prompts of unequal length at once."""
    from nanovllm import LLM, SamplingParams
    path, cfg, tensors = model_dir(tmp_path_factory, "b")
    llm = LLM(path, dtype="float32", kvcache_block_size=16, num_kvcache_blocks=40, max_num_seqs=4, max_model_len=128,
              max_num_batched_tokens=512)
    prompts = [tokens_of(cfg, n, 20 + n) for n in (9, 30, 17)]
    outs = llm.generate(prompts, SamplingParams(temperature=1.0, max_tokens=12, ignore_eos=True, greedy=True),
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


@pytest.mark.parametrize("taps,bias,act", [(2, False, None), (4, True, "silu"), (8, False, None), (1, True, None)])
def test_causal_conv_with_carried_tail(taps, bias, act):
    """Two sequences in slots 3 and 1, fed in portions of 1..40 tokens: equals the convolution of each whole
    sequence; a slot that held another sequence's tail is ignored at position 0."""
    from nanovllm import ops
    g = torch.Generator().manual_seed(taps)
    C, lens = 37, [61, 23]
    w = torch.randn(C, taps, generator=g)
    b = torch.randn(C, generator=g) if bias else None
    xs = [torch.randn(n, C, generator=g) for n in lens]
    want = []
    for x in xs:
        y = O.causal_conv(x.to(F64), w.to(F64), None if b is None else b.to(F64))
        want.append(O.silu(y) if act else y)
    state = torch.full((5, max(taps - 1, 1), C), 7.0).cuda()[:, :taps - 1].contiguous() if taps > 1 else None
    slots = torch.tensor([3, 1], dtype=torch.int32).cuda()
    got = [[], []]
    at = [0, 0]
    for portion in ([1, 2], [2, 1], [40, 3], [3, 17], [15, 0]):
        q = [min(p, lens[i] - at[i]) for i, p in enumerate(portion)]
        if q[1] == 0:
            sp, sl, parts = _spans(q[:1], [at[0] + q[0]]), slots[:1], [xs[0][at[0]:at[0] + q[0]]]
        else:
            sp, sl = _spans(q, [at[0] + q[0], at[1] + q[1]]), slots
            parts = [xs[i][at[i]:at[i] + q[i]] for i in range(2)]
        out = ops.causal_conv(_dev(torch.cat(parts)), _dev(w), None if b is None else _dev(b), sp, state, sl, act)
        got[0].append(out[:q[0]].cpu())
        if q[1]:
            got[1].append(out[q[0]:].cpu())
        at = [at[i] + q[i] for i in range(2)]
    assert at == lens
    for i in range(2):
        assert (torch.cat(got[i]).to(F64) - want[i]).abs().max() < 1e-4


def test_unitnorm_temperature_and_scatter():
    """Positions just below, at and above the multiples of the temperature's period; K and V land at their slots."""
    from nanovllm import ops
    g = torch.Generator().manual_seed(0)
    H, G, d, dv, every, coef, eps = 3, 2, 20, 12, 6, 0.9, 1e-3
    pos = torch.tensor([0, 4, 5, 6, 10, 11, 12, 35, 36, 1000])
    T = len(pos)
    qkv = torch.randn(T, H * d + G * d + G * dv, generator=g)
    q = O.rms_unit(qkv[:, :H * d].to(F64).view(T, H, d), eps)
    q = q * (1 + coef * torch.log(torch.floor((pos.to(F64) + 1) / every) + 1))[:, None, None]
    k = O.rms_unit(qkv[:, H * d:(H + G) * d].to(F64).view(T, G, d), eps)
    kc, vc = torch.zeros(4, 8, G * d).cuda(), torch.zeros(4, 8, G * dv).cuda()
    slots = torch.tensor([3, 9, 31, 0, 8, 15, 16, 17, 24, 7], dtype=torch.int32).cuda()
    buf = _dev(qkv)
    ops.unitnorm_temp_cache(buf, pos.cuda(), eps, coef, every, H, G, d, dv, kc, vc, slots)
    assert (buf[:, :H * d].cpu().to(F64) - q.reshape(T, -1)).abs().max() < 1e-5
    assert (kc.view(32, -1)[slots.long()].cpu().to(F64) - k.reshape(T, -1)).abs().max() < 1e-5
    assert torch.equal(vc.view(32, -1)[slots.long()].cpu(), qkv[:, (H + G) * d:])
    assert float(kc.abs().sum(-1).view(-1).count_nonzero()) == T


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_attention_one_key_stands_out(dtype):
    """Paged cache with a shuffled block table, 700 keys, block size 16. For chosen key positions (the first
    token, both sides of block borders, far back, the newest) the query is made to point at that key alone: the
    output must be that key's value. A key one past the causal limit must NOT be seen: the query then points at a
    key that lies just outside, and the output must stay away from its value."""
    from nanovllm import ops
    g = torch.Generator().manual_seed(1)
    H, G, d, dv, bs, n = 4, 2, 24, 40, 16, 700
    k = torch.nn.functional.normalize(torch.randn(n, G, d, generator=g), dim=-1)
    v = torch.randn(n, G, dv, generator=g)
    nblk = -(-n // bs)
    table = torch.randperm(nblk + 5, generator=g)[:nblk].to(torch.int32)
    kc, vc = torch.zeros(nblk + 5, bs, G * d), torch.zeros(nblk + 5, bs, G * dv)
    for j in range(n):
        kc[table[j // bs], j % bs] = k[j].reshape(-1)
        vc[table[j // bs], j % bs] = v[j].reshape(-1)
    kc, vc, bt = kc.to(dtype).cuda(), vc.to(dtype).cuda(), table.view(1, -1).cuda()
    tol = 2e-3 if dtype == torch.float32 else 3e-2
    for q_len in (1, 5):                               # a decoded token; the last 5 tokens of a prompt portion
        first = n - q_len
        for target in (0, 1, 15, 16, 17, 31, 32, 300, 639, 640, n - q_len - 1, n - q_len, n - 1):
            q = torch.zeros(q_len, H, d)
            for i in range(q_len):
                for h in range(H):
                    q[i, h] = 60.0 * k[target, h // (H // G)]
            sp = _spans([q_len], [n]) if q_len > 1 else ops.StepSpans(None, None, torch.tensor([n], dtype=torch.int32).cuda())
            out = ops.attn_generic(q.to(dtype).cuda(), kc, vc, sp, 1.0, G, dv, block_tables=bt).float().cpu().view(q_len, H, dv)
            for i in range(q_len):
                visible = target <= first + i
                for h in range(H):
                    err = float((out[i, h] - v[target, h // (H // G)].to(dtype).float()).abs().max())
                    assert (err < tol) == visible, (q_len, target, i, h, err)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_attention_generic_matches_plain_softmax(dtype):
    """Packed keys, three sequences of unequal length in one launch, 5 query heads per kv head."""
    from nanovllm import ops
    g = torch.Generator().manual_seed(2)
    H, G, d, dv, lens = 10, 2, 36, 20, [50, 1, 19]
    q = torch.randn(sum(lens), H, d, generator=g).to(dtype)
    k = torch.randn(sum(lens), G, d, generator=g).to(dtype)
    v = torch.randn(sum(lens), G, dv, generator=g).to(dtype)
    got = ops.attn_generic(q.cuda(), k.cuda(), v.cuda(), _spans(lens, lens), 0.2, G, dv).float().cpu()
    at = 0
    for n in lens:
        want = O.softmax_attention(q[at:at + n].to(F64), k[at:at + n].to(F64), v[at:at + n].to(F64), 0.2)
        assert (got[at:at + n].to(F64) - want.reshape(n, -1)).abs().max() < (1e-5 if dtype == torch.float32 else 2e-2)
        at += n


def test_decay_recurrence_far_token_survives():
    """A decay of 0.999 keeps a token 500 steps back visible while 0.5 has forgotten it: k of token 3 is made
    orthogonal to all others, q of the last token points at it. Fed as 40-token portions then single tokens."""
    from nanovllm import ops
    g = torch.Generator().manual_seed(3)
    H, d, dv, n = 2, 48, 24, 520
    k = torch.randn(n, H, d, generator=g) * 0.05
    k[:, :, 0] = 0
    k[3] = 0
    k[3, :, 0] = 1.0
    q = torch.randn(n, H, d, generator=g) * 0.05
    q[-1] = 0
    q[-1, :, 0] = 1.0
    v = torch.randn(n, H, dv, generator=g)
    decay = torch.tensor([0.999, 0.5])
    want = O.decay_recurrence(q.to(F64), k.to(F64), v.to(F64), decay.to(F64))
    state = torch.full((3, H, d, dv), 5.0).cuda()
    slot = torch.tensor([2], dtype=torch.int32).cuda()
    outs, at = [], 0
    for step in [40] * 12 + [1] * 40:
        sp = _spans([step], [at + step]) if step > 1 else ops.StepSpans(None, None, torch.tensor([at + 1], dtype=torch.int32).cuda())
        sl = slice(at, at + step)
        outs.append(ops.linear_recurrence(_dev(q[sl].reshape(step, -1)), _dev(k[sl].reshape(step, -1)),
                                          _dev(v[sl].reshape(step, -1)), sp, H, H, d, dv, state, slot, decay=decay.cuda()).cpu())
        at += step
    got = torch.cat(outs).view(n, H, dv)
    assert (got.to(F64) - want).abs().max() < 1e-4
    assert float((got[-1, 0] - 0.999 ** (n - 4) * v[3, 0]).abs().max()) < 1e-4      # still there
    assert float(got[-1, 1].abs().max()) < 1e-6                                      # long gone


@pytest.mark.parametrize("H,G,N,dv", [(4, 2, 20, 12), (6, 1, 64, 40), (2, 2, 130, 33)])
def test_selective_recurrence(H, G, N, dv):
    from nanovllm import ops
    g = torch.Generator().manual_seed(H)
    lens = [33, 9]
    T = sum(lens)
    x, B, C = torch.randn(T, H, dv, generator=g), torch.randn(T, G, N, generator=g), torch.randn(T, G, N, generator=g)
    dt = torch.randn(T, H, generator=g) * 2
    dt[5] = 30.0                                         # softplus far in its linear range
    dt_bias, A_log, D = torch.randn(H, generator=g), torch.rand(H, generator=g) * 2 - 2, torch.randn(H, generator=g)
    got = []
    state = torch.zeros(2, H, N, dv).cuda()
    slots = torch.tensor([1, 0], dtype=torch.int32).cuda()
    at = [0, lens[0]]
    for portion in ([20, 2], [13, 7]):
        idx = torch.cat([torch.arange(at[i], at[i] + portion[i]) for i in range(2)])
        done = [at[0] + portion[0], at[1] - lens[0] + portion[1]]
        out = ops.linear_recurrence(_dev(C[idx].reshape(len(idx), -1)), _dev(B[idx].reshape(len(idx), -1)),
                                    _dev(x[idx].reshape(len(idx), -1)), _spans(portion, done), H, G, N, dv, state, slots,
                                    dt=_dev(dt[idx]), dt_bias=_dev(dt_bias), a_log=_dev(A_log), d_skip=_dev(D)).cpu()
        got.append((idx, out))
        at = [at[i] + portion[i] for i in range(2)]
    full = torch.zeros(T, H * dv)
    for idx, out in got:
        full[idx] = out
    lo = 0
    for n in lens:
        s = slice(lo, lo + n)
        step = torch.nn.functional.softplus(dt[s].to(F64) + dt_bias.to(F64), threshold=1e9)
        want = O.selective_scan(x[s].to(F64), B[s].to(F64), C[s].to(F64), step, A_log.to(F64), D.to(F64))
        assert (full[s].to(F64) - want.reshape(n, -1)).abs().max() < 2e-4 * want.abs().max()
        lo += n


@pytest.mark.parametrize("H,G,N,dv,mode", [(2, 2, 128, 64, "selective"), (3, 1, 20, 12, "selective"),
                                             (2, 2, 64, 128, "decay"), (4, 4, 24, 40, "decay")])
def test_recurrence_sixteen_tokens_at_a_time(H, G, N, dv, mode):
    """bf16 prompt portions run on the tensor cores, 16 tokens per step with every fp32 operand split into three
    bf16 terms: the result must agree with the token-by-token recurrence to fp32 accuracy (the inputs are bf16
    values, so the float64 oracle sees exactly the same numbers). Portions of 40, 17, 16 and 33 tokens cross the
    16-token steps at every offset; a second sequence of one long portion shares the launches; then single tokens."""
    from nanovllm import ops
    g = torch.Generator().manual_seed(N + dv)
    bf = torch.bfloat16
    lens = [40 + 17 + 16 + 33 + 3, 90]
    T = sum(lens)
    q = (torch.randn(T, G, N, generator=g) * 0.3).to(bf)
    k = (torch.randn(T, G, N, generator=g) * 0.3).to(bf)
    v = torch.randn(T, H, dv, generator=g).to(bf)
    state = torch.full((3, H, N, dv), 9.0).cuda()
    slots = torch.tensor([2, 0], dtype=torch.int32).cuda()
    if mode == "decay":
        assert G == H
        decay = torch.tensor([0.999, 0.9, 0.5, 0.97][:H])
        kw = dict(decay=decay.cuda())
    else:
        dt = (torch.randn(T, H, generator=g)).to(bf)
        dt_bias, A_log, D = torch.randn(H, generator=g), torch.rand(H, generator=g) * 2 - 2, torch.randn(H, generator=g)
        kw = dict(dt_bias=dt_bias.cuda(), a_log=A_log.cuda(), d_skip=D.cuda())
    full = torch.zeros(T, H * dv)
    at = [0, 0]
    for portion in ([40, 90], [17, 0], [16, 0], [33, 0], [1, 0], [1, 0], [1, 0]):
        idx = torch.cat([torch.arange(at[0], at[0] + portion[0]), lens[0] + torch.arange(at[1], at[1] + portion[1])])
        qs = [p for p in portion if p]
        ks = [a + p for a, p in zip(at, portion) if p]
        if qs == [1]:
            sp = ops.StepSpans(None, None, torch.tensor(ks, dtype=torch.int32).cuda())
        else:
            sp = _spans(qs, ks)
        extra = dict(kw, dt=dt[idx].cuda()) if mode == "selective" else kw
        out = ops.linear_recurrence(q[idx].reshape(len(idx), -1).cuda(), k[idx].reshape(len(idx), -1).cuda(),
                                    v[idx].reshape(len(idx), -1).cuda(), sp, H, G, N, dv, state, slots[:len(qs)],
                                    **extra).cpu()
        full[idx] = out
        at = [a + p for a, p in zip(at, portion)]
    assert at == lens
    lo = 0
    for n in lens:
        sl = slice(lo, lo + n)
        if mode == "decay":
            want = O.decay_recurrence(q[sl].to(F64), k[sl].to(F64), v[sl].to(F64), decay.to(F64))
        else:
            step = torch.nn.functional.softplus(dt[sl].to(F64) + dt_bias.to(F64), threshold=1e9)
            want = O.selective_scan(v[sl].to(F64), k[sl].to(F64), q[sl].to(F64), step, A_log.to(F64), D.to(F64))
        assert (full[sl].to(F64) - want.reshape(n, -1)).abs().max() < 1e-4 * want.abs().max(), (mode, lo)
        lo += n


def test_gated_norms_and_feed_forward_activation():
    from nanovllm import ops
    g = torch.Generator().manual_seed(4)
    rows, n, eps = 7, 60, 1e-4
    y, gate, w = torch.randn(rows, n, generator=g) * 3, torch.randn(rows, n + 5, generator=g), torch.randn(n, generator=g)
    gd = _dev(gate)[:, 5:]
    a = ops.gated_norm(_dev(y), gd, _dev(w), eps, 1, False, "sigmoid").cpu().to(F64)
    want = O.rms_unit(y.to(F64), eps) * w.to(F64) * torch.sigmoid(gate[:, 5:].to(F64))
    assert (a - want).abs().max() < 1e-5
    b = ops.gated_norm(_dev(y), gd, _dev(w), eps, 4, True, "silu").cpu().to(F64)
    z = y.to(F64) * O.silu(gate[:, 5:].to(F64))
    want = O.rms_unit(z.view(rows, 4, n // 4), eps).reshape(rows, n) * w.to(F64)
    assert (b - want).abs().max() < 1e-5
    c = ops.gated_norm(_dev(y), gd, None, eps).cpu().to(F64)
    assert (c - y.to(F64) * torch.sigmoid(gate[:, 5:].to(F64))).abs().max() < 1e-5
    x = torch.randn(rows, 2 * 33, generator=g) * 2
    for act, fn in (("relu", torch.relu), ("silu", O.silu), ("gelu_tanh", O.gelu_tanh)):
        got = ops.act_and_mul(_dev(x), act).cpu().to(F64)
        assert (got - fn(x[:, :33].to(F64)) * x[:, 33:].to(F64)).abs().max() < 1e-5, act


def test_residual_norms():
    from nanovllm import ops
    g = torch.Generator().manual_seed(5)
    rows, n, eps = 5, 77, 1e-6
    r, y = torch.randn(rows, n, generator=g) * 4, torch.randn(rows, n, generator=g)
    w1, w2 = torch.randn(n, generator=g) * 0.2, torch.randn(n, generator=g) * 0.2
    h0 = ops.residual_rmsnorm(_dev(r), _dev(w1), eps, torch.float32).cpu().to(F64)
    assert (h0 - O.norm_offset(r.to(F64), w1.to(F64), eps)).abs().max() < 1e-5
    rd = _dev(r)
    h = ops.residual_add_norms_(_dev(y), rd, _dev(w1), _dev(w2), eps).cpu().to(F64)
    r2 = r.to(F64) + O.norm_offset(y.to(F64), w1.to(F64), eps)
    assert (rd.cpu().to(F64) - r2).abs().max() < 1e-5
    assert (h - O.norm_offset(r2, w2.to(F64), eps)).abs().max() < 1e-5
    assert ops.residual_add_norms_(_dev(y), rd, _dev(w1), None, eps) is None
