"""Plain, slow restatement of the Nirelix decoder for the tests: one function per mechanism, token by
token where the mechanism is a recurrence, float64 on the CPU. It shares no code with the package.

Notation: ``u`` is a sublayer's input [T, width]; weights are stored [out, in] and applied as ``u @ W.T``.
A model is (config dict, {tensor name: float64 tensor}) with the checkpoint's names (``l<i>.mix.q`` ...).
"""
from __future__ import annotations

import math

import torch

F64 = torch.float64


# ----------------------------------------------------------------------------- small pieces
def rms_unit(x, eps):
    return x / torch.sqrt(x.pow(2).mean(-1, keepdim=True) + eps)


def layer_norm(x, w, b, eps):
    mu = x.mean(-1, keepdim=True)
    var = (x - mu).pow(2).mean(-1, keepdim=True)
    return (x - mu) / torch.sqrt(var + eps) * w + b


def silu(x):
    return x * torch.sigmoid(x)


def softplus(x):
    return torch.where(x > 30, x, torch.log1p(torch.exp(torch.clamp(x, max=30.0))))


def causal_conv(u, w):
    """u [T, C], w [C, taps]; the last column of w multiplies the current token, zeros before t = 0."""
    T, _ = u.shape
    taps = w.shape[1]
    out = torch.zeros_like(u)
    for t in range(T):
        for j in range(taps):
            s = t - taps + 1 + j
            if s >= 0:
                out[t] += w[:, j] * u[s]
    return out


def rotate(x, pos, dims, base, interleaved):
    """x [T, H, d]; the first ``dims`` entries of each head are rotated by angle pos * base^(-2i/dims) in pairs
    (2i, 2i+1) when ``interleaved`` else (i, i + dims/2)."""
    out = x.clone()
    half = dims // 2
    for i in range(half):
        f = float(base) ** (-2.0 * i / dims)
        a, b = (2 * i, 2 * i + 1) if interleaved else (i, i + half)
        ang = pos.to(F64) * f
        c, s = torch.cos(ang)[:, None], torch.sin(ang)[:, None]
        p, r = x[..., a], x[..., b]
        out[..., a] = p * c - r * s
        out[..., b] = r * c + p * s
    return out


# ----------------------------------------------------------------------------- mixers
def retention_recurrence(q, k, v, decay):
    """S <- decay_h S + k v^T; o = S^T q. q, k [T, H, d]; v [T, H, dv]."""
    T, H, d = q.shape
    dv = v.shape[2]
    S = torch.zeros(H, d, dv, dtype=q.dtype)
    out = torch.zeros(T, H, dv, dtype=q.dtype)
    for t in range(T):
        for h in range(H):
            S[h] = decay[h] * S[h] + torch.outer(k[t, h], v[t, h])
            out[t, h] = S[h].T @ q[t, h]
    return out


def retention_mixer(u, P, m, eps):
    T = u.shape[0]
    H, d, dv = m["heads"], m["dim"], m["vdim"]
    pos = torch.arange(T)
    q = rotate((u @ P["q"].T).view(T, H, d), pos, m["rot"]["dims"], m["rot"]["base"], False)
    k = rotate((u @ P["k"].T).view(T, H, d), pos, m["rot"]["dims"], m["rot"]["base"], False) * d ** -0.5
    v = (u @ P["v"].T).view(T, H, dv)
    o = retention_recurrence(q, k, v, [float(x) for x in m["decay"]])
    o = rms_unit(o, eps).reshape(T, H * dv)
    return (o * silu(u @ P["g"].T)) @ P["o"].T


def delta_recurrence(q, k, v, g, beta):
    """Per head: S <- g (rows) * S; w = beta (v - S^T k); S <- S + k w^T; o = S^T q.
    q, k, g [T, H, d]; v [T, H, dv]; beta [T, H]."""
    T, H, d = q.shape
    dv = v.shape[2]
    S = torch.zeros(H, d, dv, dtype=q.dtype)
    out = torch.zeros(T, H, dv, dtype=q.dtype)
    for t in range(T):
        for h in range(H):
            S[h] = g[t, h][:, None] * S[h]
            w = beta[t, h] * (v[t, h] - S[h].T @ k[t, h])
            S[h] = S[h] + torch.outer(k[t, h], w)
            out[t, h] = S[h].T @ q[t, h]
    return out


def channel_delta_mixer(u, P, m, eps):
    T = u.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = silu(causal_conv(u @ P["q"].T, P["q.conv"])).view(T, G, d)
    k = silu(causal_conv(u @ P["k"].T, P["k.conv"])).view(T, G, d)
    v = silu(causal_conv(u @ P["v"].T, P["v.conv"])).view(T, H, dv)
    q = q / torch.sqrt(q.pow(2).sum(-1, keepdim=True) + 1e-6) * d ** -0.5
    k = k / torch.sqrt(k.pow(2).sum(-1, keepdim=True) + 1e-6)
    rep = H // G
    q = q.repeat_interleave(rep, 1)
    k = k.repeat_interleave(rep, 1)
    beta = torch.sigmoid(u @ P["b"].T)
    a = ((u @ P["a1"].T) @ P["a2"].T + P["dt_bias"]).view(T, H, d)
    g = torch.exp(-torch.exp(P["A_log"])[None, :, None] * softplus(a))
    o = delta_recurrence(q, k, v, g, beta)
    o = rms_unit(o, eps) * P["norm"]
    gate = torch.sigmoid((u @ P["g1"].T) @ P["g2"].T).view(T, H, dv)
    return (o * gate).reshape(T, H * dv) @ P["o"].T


def latent_attention_mixer(u, P, m, eps):
    T = u.shape[0]
    H, d, dr, dv, R = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    pos = torch.arange(T)
    cq = rms_unit(u @ P["dq"].T, eps) * P["dq.norm"]
    q = (cq @ P["uq"].T).view(T, H, d + dr)
    kv = u @ P["dkv"].T
    c = rms_unit(kv[:, :R], eps) * P["dkv.norm"]
    kr = rotate(kv[:, None, R:], pos, m["rot"]["dims"], m["rot"]["base"], True)[:, 0]
    qr = rotate(q[..., d:], pos, m["rot"]["dims"], m["rot"]["base"], True)
    kn = (c @ P["uk"].T).view(T, H, d)
    val = (c @ P["uv"].T).view(T, H, dv)
    out = torch.zeros(T, H, dv, dtype=u.dtype)
    W = (m.get("mask") or {}).get("size") or T + 1          # no mask entry: plain causal attention
    for i in range(T):
        lo = max(0, i - W + 1)
        for h in range(H):
            s = (kn[lo:i + 1, h] @ q[i, h, :d] + kr[lo:i + 1] @ qr[i, h]) * m["scale"]
            out[i, h] = torch.softmax(s, 0) @ val[lo:i + 1, h]
    return (out.reshape(T, H * dv) * torch.sigmoid(u @ P["g"].T)) @ P["o"].T


MIXERS = {"retention": retention_mixer, "channel_delta": channel_delta_mixer, "latent_attention": latent_attention_mixer}


# ----------------------------------------------------------------------------- feed-forward
def dense_ff(u, P, limit):
    g = torch.clamp(u @ P["gate"].T, max=limit)
    up = torch.clamp(u @ P["up"].T, -limit, limit)
    return (g * torch.sigmoid(1.702 * g) * (up + 1.0)) @ P["down"].T


def route(z, correction, r):
    """z [T, E] router logits -> (chosen [T, top], weights [T, top])."""
    T, E = z.shape
    s = torch.sigmoid(z)
    choice = s + correction
    grp_cfg = r.get("groups") or {"count": 1, "keep": 1}
    n, keep, top = grp_cfg["count"], grp_cfg["keep"], r["top"]
    per = E // n
    grp = choice.view(T, n, per)
    gscore = grp.topk(min(2, per), -1).values.sum(-1)
    best = gscore.topk(keep, -1).indices
    allowed = torch.zeros(T, n, dtype=torch.bool)
    allowed.scatter_(1, best, True)
    masked = torch.where(allowed[:, :, None].expand(T, n, per).reshape(T, E), choice,
                         torch.full_like(choice, -math.inf))
    idx = masked.topk(top, -1).indices
    w = s.gather(1, idx)
    w = w / (w.sum(-1, keepdim=True) + 1e-20) * r.get("scale", 1.0)
    return idx, w


def moe_ff(u, P, mlp):
    r = mlp["router"]
    idx, w = route(u @ P["router"].T, P["correction"], r)
    out = torch.zeros_like(u)
    for t in range(u.shape[0]):
        for j in range(idx.shape[1]):
            e = int(idx[t, j])
            h = silu(u[t] @ P[f"e{e}.gate"].T) * (u[t] @ P[f"e{e}.up"].T)
            out[t] += w[t, j] * (h @ P[f"e{e}.down"].T)
    return out


def feed_forward(u, P, mlp):
    return dense_ff(u, P, mlp["limit"]) if mlp["kind"] == "dense" else moe_ff(u, P, mlp)


# ----------------------------------------------------------------------------- the model
def sub(tensors, prefix):
    return {k[len(prefix):]: v for k, v in tensors.items() if k.startswith(prefix)}


def hyper_step(X, hc, fn):
    """X [S, T, W] streams; hc has 'in' [S], 'out' [S], 'mix' [S(from), S(to)]."""
    u = torch.einsum("s,stw->tw", hc["in"], X)
    y = fn(u)
    return torch.einsum("st,snw->tnw", hc["mix"], X) + hc["out"][:, None, None] * y[None]


def forward(config, tensors, tokens, return_layers=False):
    eps = config["norm"]["eps"]
    S = config.get("streams", 1)
    x = tensors["embed"][torch.as_tensor(tokens)]
    X = x[None].repeat(S, 1, 1)
    layers = []
    ones = {"in": torch.ones(1, dtype=F64), "out": torch.ones(1, dtype=F64), "mix": torch.ones(1, 1, dtype=F64)}
    for i, entry in enumerate(config["layers"]):
        T_ = sub(tensors, f"l{i}.")
        hc1 = sub(T_, "hc1.") if "streams" in config else ones
        hc2 = sub(T_, "hc2.") if "streams" in config else ones
        X = hyper_step(X, hc1, lambda u: MIXERS[entry["type"]](
            layer_norm(u, T_["norm1"], T_["norm1.b"], eps), sub(T_, "mix."), entry["mixer"], eps))
        if entry.get("mlp"):
            X = hyper_step(X, hc2, lambda u: feed_forward(
                layer_norm(u, T_["norm2"], T_["norm2.b"], eps), sub(T_, "mlp."), entry["mlp"]))
        layers.append(X.sum(0))
    h = layer_norm(X.sum(0), tensors["final.norm"], tensors["final.norm.b"], eps)
    logits = h @ tensors["head"].T
    return (logits, torch.stack(layers)) if return_layers else logits


def random_model(config, seed=0, ranks=(5, 3)):
    """Random bf16-representable weights for `config` under the checkpoint's names and shapes, returned as
    {name: bf16 tensor}. `ranks`: inner sizes of the delta mixers' low-rank decay and gate projections."""
    g = torch.Generator().manual_seed(seed)
    W, V, S = config["width"], config["vocab"], config.get("streams")
    t = {}

    def mat(name, out, inn, s=None):
        t[name] = (torch.randn(out, inn, generator=g) * (s if s is not None else inn ** -0.5)).bfloat16()

    def vec(name, n, s=0.1, mean=0.0):
        t[name] = (mean + torch.randn(n, generator=g) * s).bfloat16()

    mat("embed", V, W, 1.0)
    for i, layer in enumerate(config["layers"]):
        p, m = f"l{i}.", layer["mixer"]
        for q in ("1", "2") if layer.get("mlp") else ("1",):
            vec(p + "norm" + q, W, mean=1.0)
            vec(p + "norm" + q + ".b", W)
            if S is not None:
                vec(p + f"hc{q}.in", S, 0.2, S ** -0.5)
                vec(p + f"hc{q}.out", S, 0.2, 1.0)
                t[p + f"hc{q}.mix"] = (torch.eye(S) + 0.15 * torch.randn(S, S, generator=g)).bfloat16()
        if layer["type"] == "retention":
            H, d, dv = m["heads"], m["dim"], m["vdim"]
            for n, rows in (("q", H * d), ("k", H * d), ("v", H * dv), ("g", H * dv)):
                mat(p + "mix." + n, rows, W)
            mat(p + "mix.o", W, H * dv)
        elif layer["type"] == "channel_delta":
            H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
            for n, rows in (("q", G * d), ("k", G * d), ("v", H * dv)):
                mat(p + "mix." + n, rows, W)
                t[p + "mix." + n + ".conv"] = (torch.randn(rows, m["conv"], generator=g) * 0.5).bfloat16()
            mat(p + "mix.b", H, W)
            t[p + "mix.A_log"] = (torch.rand(H, generator=g) * 3 - 4).bfloat16()
            vec(p + "mix.norm", dv, mean=1.0)
            mat(p + "mix.a1", ranks[0], W)
            mat(p + "mix.a2", H * d, ranks[0], 1.0)
            vec(p + "mix.dt_bias", H * d, 1.0)
            mat(p + "mix.g1", ranks[1], W)
            mat(p + "mix.g2", H * dv, ranks[1], 1.0)
            mat(p + "mix.o", W, H * dv)
        else:
            H, d, dr, dv, R, Q = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"], m["q_rank"]
            mat(p + "mix.dq", Q, W)
            vec(p + "mix.dq.norm", Q, mean=1.0)
            mat(p + "mix.uq", H * (d + dr), Q)
            mat(p + "mix.dkv", R + dr, W)
            vec(p + "mix.dkv.norm", R, mean=1.0)
            mat(p + "mix.uk", H * d, R)
            mat(p + "mix.uv", H * dv, R)
            mat(p + "mix.g", H * dv, W)
            mat(p + "mix.o", W, H * dv)
        mlp = layer.get("mlp")
        if mlp and mlp["kind"] == "dense":
            mat(p + "mlp.gate", mlp["ff"], W, 2.0 * W ** -0.5)
            mat(p + "mlp.up", mlp["ff"], W, 2.0 * W ** -0.5)
            mat(p + "mlp.down", W, mlp["ff"])
        elif mlp:
            E, ff = mlp["router"]["experts"], mlp["expert"]["ff"]
            for e in range(E):
                mat(p + f"mlp.e{e}.gate", ff, W)
                mat(p + f"mlp.e{e}.up", ff, W)
                mat(p + f"mlp.e{e}.down", W, ff)
            mat(p + "mlp.router", E, W, 2.0 * W ** -0.5)
            vec(p + "mlp.correction", E, 0.5, -0.3)
    vec("final.norm", W, mean=1.0)
    vec("final.norm.b", W)
    mat("head", V, W)
    return t


def as_f64(tensors):
    return {k: v.to(F64) for k, v in tensors.items()}
