"""Plain, slow restatement of the Zegopel decoder for the tests: one function per mechanism, token by
token where the mechanism is a recurrence, float64 on the CPU. It shares no code with the package.

Notation: ``u`` is a sublayer's input [T, width]; weights are stored [out, in] and applied as ``u @ W.T``.
A model is (config dict, {tensor name: tensor}) with the checkpoint's names (``l<i>.mix.q`` ...).
"""
from __future__ import annotations

import math

import torch

F64 = torch.float64


def rms_unit(x, eps):
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / torch.sqrt(x.pow(2).mean(-1, keepdim=True) + eps)


def norm_offset(x, w, eps):
    """RMS norm whose stored weight is the deviation from one."""
    return rms_unit(x, eps) * (1.0 + w)


def silu(x):
    return x * torch.sigmoid(x)


def gelu_tanh(x):
    return 0.5 * x * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (x + 0.044715 * x ** 3)))


def causal_conv(u, w, bias=None):
    """u [T, C], w [C, taps]; the last column of w multiplies the current token, zeros before t = 0."""
    T, C = u.shape
    taps = w.shape[1]
    out = torch.zeros(T, C, dtype=u.dtype)
    for t in range(T):
        for j in range(taps):
            s = t - taps + 1 + j
            if s >= 0:
                out[t] += w[:, j] * u[s]
    return out if bias is None else out + bias


def softmax_attention(q, k, v, scale):
    """q [T, H, d], k [T, G, d], v [T, G, dv]; causal; query head h reads kv head h // (H / G)."""
    T, H, _ = q.shape
    G = k.shape[1]
    out = torch.zeros(T, H, v.shape[2], dtype=q.dtype)
    for h in range(H):
        g = h // (H // G)
        for i in range(T):
            s = (k[: i + 1, g] @ q[i, h]) * scale
            p = torch.softmax(s, 0)
            out[i, h] = p @ v[: i + 1, g]
    return out


def attention_mixer(u, P, m, eps):
    """P: tensors of this mixer by short name ('q', 'q.b', 'q.conv', ..., 'g', 'o')."""
    T = u.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = causal_conv(u @ P["q"].T + P["q.b"], P["q.conv"])
    k = causal_conv(u @ P["k"].T + P["k.b"], P["k.conv"])
    v = causal_conv(u @ P["v"].T + P["v.b"], P["v.conv"])
    q = rms_unit(q.view(T, H, d), eps)
    k = rms_unit(k.view(T, G, d), eps)
    pos = torch.arange(T, dtype=F64)
    every, coef = m["q_temp"]["every"], m["q_temp"]["coef"]
    temp = 1.0 + coef * torch.log(torch.floor((pos + 1) / every) + 1.0)
    q = q * temp[:, None, None]
    o = softmax_attention(q, k, v.view(T, G, dv), m["scale"]).reshape(T, H * dv)
    return (o * torch.sigmoid(u @ P["g"].T)) @ P["o"].T


def decay_recurrence(q, k, v, decay):
    """Per head S <- decay_h S + k v^T, o = S^T q. q, k [T, H, d]; v [T, H, dv]; decay [H]."""
    T, H, d = q.shape
    dv = v.shape[2]
    S = torch.zeros(H, d, dv, dtype=q.dtype)
    out = torch.zeros(T, H, dv, dtype=q.dtype)
    for t in range(T):
        S = decay[:, None, None] * S + k[t, :, :, None] * v[t, :, None, :]
        out[t] = torch.einsum("hkv,hk->hv", S, q[t])
    return out


def lightning_mixer(u, P, m, eps):
    T = u.shape[0]
    H, d, dv = m["heads"], m["dim"], m["vdim"]
    q = silu(u @ P["q"].T).view(T, H, d)
    k = silu(u @ P["k"].T).view(T, H, d)
    v = silu(u @ P["v"].T).view(T, H, dv)
    o = decay_recurrence(q, k, v, torch.tensor(m["decay"], dtype=F64)).reshape(T, H * dv)
    o = rms_unit(o, eps) * P["norm"]
    return (o * torch.sigmoid(u @ P["g"].T)) @ P["o"].T


def selective_scan(x, B, C, dt, A_log, D):
    """x [T, H, dv], B and C [T, G, N], dt [T, H] (after softplus). S is [N, dv] per head."""
    T, H, dv = x.shape
    G, N = B.shape[1], B.shape[2]
    S = torch.zeros(H, N, dv, dtype=x.dtype)
    y = torch.zeros(T, H, dv, dtype=x.dtype)
    rate = torch.exp(A_log)
    for t in range(T):
        for h in range(H):
            g = h // (H // G)
            S[h] = torch.exp(-rate[h] * dt[t, h]) * S[h] + dt[t, h] * B[t, g][:, None] * x[t, h][None, :]
            y[t, h] = S[h].T @ C[t, g] + D[h] * x[t, h]
    return y


def mamba2_mixer(u, P, m, eps):
    T = u.shape[0]
    H, dv, N, G = m["heads"], m["vdim"], m["state"], m["groups"]
    inner = H * dv
    proj = u @ P["in"].T
    z, xbc, dt = proj[:, :inner], proj[:, inner:2 * inner + 2 * G * N], proj[:, 2 * inner + 2 * G * N:]
    xbc = silu(causal_conv(xbc, P["conv"], P["conv.b"]))
    x = xbc[:, :inner].reshape(T, H, dv)
    B = xbc[:, inner:inner + G * N].reshape(T, G, N)
    C = xbc[:, inner + G * N:].reshape(T, G, N)
    dt = torch.nn.functional.softplus(dt + P["dt_bias"], threshold=1e9)
    y = selective_scan(x, B, C, dt, P["A_log"], P["D"]).reshape(T, inner)
    y = y * silu(z)
    parts = m["norm_groups"]
    y = rms_unit(y.view(T, parts, inner // parts), eps).reshape(T, inner) * P["norm"]
    return y @ P["o"].T


def feed_forward(u, P, act="relu"):
    fn = {"relu": torch.relu, "silu": silu, "gelu_tanh": gelu_tanh}[act]
    return (fn(u @ P["gate"].T) * (u @ P["up"].T)) @ P["down"].T


MIXERS = {"attention": attention_mixer, "lightning": lightning_mixer, "mamba2": mamba2_mixer}


def sub(tensors, prefix):
    return {k[len(prefix):]: v.to(F64) for k, v in tensors.items() if k.startswith(prefix)}


def forward(config, tensors, tokens, return_layers=False):
    """Logits [T, vocab] of one sequence (float64); optionally the residual stream after each layer."""
    eps = config["norm"]["eps"]
    x = tensors["embed"].to(F64)[torch.as_tensor(tokens)]
    layers = []
    for i, layer in enumerate(config["layers"]):
        p = f"l{i}."
        w = lambda n: tensors[p + n].to(F64)
        y = MIXERS[layer["type"]](norm_offset(x, w("norm1"), eps), sub(tensors, p + "mix."), layer["mixer"], eps)
        x = x + norm_offset(y, w("norm1b"), eps)
        if layer.get("mlp"):
            y = feed_forward(norm_offset(x, w("norm2"), eps), sub(tensors, p + "mlp."),
                             layer["mlp"].get("act", "relu"))
            x = x + norm_offset(y, w("norm2b"), eps)
        layers.append(x)
    logits = norm_offset(x, tensors["final.norm"].to(F64), eps) @ tensors["head"].to(F64).T
    return (logits, torch.stack(layers)) if return_layers else logits


def random_model(config, seed=0, std=None):
    """Random bf16-representable weights for `config` (checkpoint names and shapes)."""
    g = torch.Generator().manual_seed(seed)
    W, V = config["width"], config["vocab"]
    t = {}

    def mat(name, out, inn, s=None):
        s = s if s is not None else (std if std is not None else inn ** -0.5)
        t[name] = (torch.randn(out, inn, generator=g) * s).bfloat16()

    def vec(name, n, s=0.1, mean=0.0):
        t[name] = (mean + torch.randn(n, generator=g) * s).bfloat16()

    mat("embed", V, W, 1.0)
    for i, layer in enumerate(config["layers"]):
        p, m = f"l{i}.", layer["mixer"]
        vec(p + "norm1", W)
        vec(p + "norm1b", W)
        if layer["type"] == "attention":
            H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
            for n, rows in (("q", H * d), ("k", G * d), ("v", G * dv)):
                mat(p + "mix." + n, rows, W)
                vec(p + "mix." + n + ".b", rows)
                t[p + "mix." + n + ".conv"] = (torch.randn(rows, m["conv"], generator=g) * 0.5).bfloat16()
            mat(p + "mix.g", H * dv, W)
            mat(p + "mix.o", W, H * dv)
        elif layer["type"] == "lightning":
            H, d, dv = m["heads"], m["dim"], m["vdim"]
            mat(p + "mix.q", H * d, W)
            mat(p + "mix.k", H * d, W)
            mat(p + "mix.v", H * dv, W)
            mat(p + "mix.g", H * dv, W)
            mat(p + "mix.o", W, H * dv)
            vec(p + "mix.norm", H * dv, mean=1.0)
        else:
            H, dv, N, G = m["heads"], m["vdim"], m["state"], m["groups"]
            inner, ch = H * dv, H * dv + 2 * G * N
            mat(p + "mix.in", 2 * inner + 2 * G * N + H, W)
            t[p + "mix.conv"] = (torch.randn(ch, m["conv"], generator=g) * 0.5).bfloat16()
            vec(p + "mix.conv.b", ch)
            vec(p + "mix.dt_bias", H, 0.5)
            t[p + "mix.A_log"] = (torch.rand(H, generator=g) * 2 - 2).bfloat16()
            vec(p + "mix.D", H, 0.5, 1.0)
            vec(p + "mix.norm", inner, mean=1.0)
            mat(p + "mix.o", W, inner)
        if layer.get("mlp"):
            ff = layer["mlp"]["ff"]
            vec(p + "norm2", W)
            vec(p + "norm2b", W)
            mat(p + "mlp.gate", ff, W)
            mat(p + "mlp.up", ff, W)
            mat(p + "mlp.down", W, ff)
    vec("final.norm", W)
    mat("head", V, W)
    return t
