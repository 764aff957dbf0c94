"""A plain float64 restatement of the Silonex design, one function per mechanism, token by token where the design is recurrent.  It shares
no code with the package: the tests build small random models, run them here and through the engine, and compare.

A model is (config, tensors): config as in config.json, tensors a dict name -> torch tensor with the checkpoint's names.

Notation: X the residual streams [streams, T, width]; y a sublayer's normed input [T, width]; p the position of a token in its sequence."""
import math

import torch

F64 = torch.float64


def d(t):
    return t.to(F64)


def layer_norm(x, w, b, eps):
    mu = x.mean(-1, keepdim=True)
    var = ((x - mu) ** 2).mean(-1, keepdim=True)
    return (x - mu) / torch.sqrt(var + eps) * w + b


def rms_unit(x, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def silu(z):
    return z * torch.sigmoid(z)


def softplus(z):
    return torch.where(z > 30.0, z, torch.log1p(torch.exp(torch.clamp(z, max=30.0))))


def causal_conv(x, w, b=None):
    """x [T, channels], w [channels, taps] (last column weighs the current token), zeros before the start."""
    T, taps = x.shape[0], w.shape[1]
    out = torch.zeros_like(x)
    for t in range(T):
        for j in range(taps):
            src = t - (taps - 1 - j)
            if src >= 0:
                out[t] += w[:, j] * x[src]
    return out if b is None else out + b


def rotary_frequencies(rot):
    """Angle per position of every pair, with the long wavelengths slowed down and a smooth band between (Llama-3.1 style)."""
    dims = rot["dims"]
    f = torch.tensor([rot["base"] ** (-2.0 * i / dims) for i in range(dims // 2)], dtype=F64)
    sc = rot.get("scaling")
    if not sc:
        return f
    out = f.clone()
    for i in range(dims // 2):
        wl = 2.0 * math.pi / float(f[i])
        if wl < sc["original"] / sc["high"]:
            continue
        if wl > sc["original"] / sc["low"]:
            out[i] = f[i] / sc["factor"]
        else:
            s = (sc["original"] / wl - sc["low"]) / (sc["high"] - sc["low"])
            out[i] = (1.0 - s) * f[i] / sc["factor"] + s * f[i]
    return out


def rotate_half(v, pos, rot):
    """v [T, heads, dim]: channel i pairs with channel i + dims/2 among the first `dims`; the rest pass unchanged."""
    dims = rot["dims"]
    if dims == 0:
        return v
    half = dims // 2
    ang = pos.to(F64)[:, None] * rotary_frequencies(rot)[None, :]
    c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    out = v.clone()
    a, b = v[..., :half], v[..., half:dims]
    out[..., :half] = a * c - b * s
    out[..., half:dims] = b * c + a * s
    return out


def mixer_lightning(y, W, mx):
    """Linear attention with one constant decay per head: S <- decay S + k v^T; o = S^T q, token by token."""
    T = y.shape[0]
    H, dk, dv = mx["heads"], mx["dim"], mx["vdim"]
    q = silu(y @ d(W["q"]).T).reshape(T, H, dk)
    k = silu(y @ d(W["k"]).T).reshape(T, H, dk)
    v = silu(y @ d(W["v"]).T).reshape(T, H, dv)
    S = torch.zeros(H, dk, dv, dtype=F64)
    o = torch.zeros(T, H, dv, dtype=F64)
    for t in range(T):
        for h in range(H):
            S[h] = mx["decay"][h] * S[h] + torch.outer(k[t, h], v[t, h])
            o[t, h] = S[h].T @ q[t, h]
    return o, q, k, v


def lightning_output(o, y, W, eps):
    T = o.shape[0]
    r = rms_unit(o.reshape(T, -1), eps) * d(W["norm"])
    return (r * torch.sigmoid(y @ d(W["g"]).T)) @ d(W["o"]).T


def mixer_mamba2(y, W, mx, eps):
    """State-space mixer: short convolution on x, B, C; a step size per head; S <- exp(-exp(A) dt) S + dt B x^T; out = S^T C + D x."""
    T = y.shape[0]
    H, P, N, G = mx["heads"], mx["vdim"], mx["state"], mx["groups"]
    inner = H * P
    proj = y @ d(W["in"]).T
    z, xbc, dt = proj[:, :inner], proj[:, inner:2 * inner + 2 * G * N], proj[:, 2 * inner + 2 * G * N:]
    xbc = silu(causal_conv(xbc, d(W["conv"]), d(W["conv.b"])))
    x = xbc[:, :inner].reshape(T, H, P)
    B = xbc[:, inner:inner + G * N].reshape(T, G, N)
    Cm = xbc[:, inner + G * N:].reshape(T, G, N)
    dt = softplus(dt + d(W["dt_bias"]))
    A = torch.exp(d(W["A_log"]))
    S = torch.zeros(H, N, P, dtype=F64)
    out = torch.zeros(T, H, P, dtype=F64)
    for t in range(T):
        for h in range(H):
            g = h // (H // G)
            S[h] = torch.exp(-A[h] * dt[t, h]) * S[h] + dt[t, h] * torch.outer(B[t, g], x[t, h])
            out[t, h] = S[h].T @ Cm[t, g] + d(W["D"])[h] * x[t, h]
    gated = out.reshape(T, inner) * silu(z)
    parts = mx["norm_groups"]
    normed = rms_unit(gated.reshape(T, parts, inner // parts), eps).reshape(T, inner) * d(W["norm"])
    return normed @ d(W["o"]).T


def mixer_window_attention(y, W, mx, eps, pos=None):
    """Grouped-query softmax attention over a sliding window: per-head q/k norm, rotation in halves, unit-RMS values, capped scores."""
    T = y.shape[0]
    H, G, dk, dv = mx["heads"], mx["kv_heads"], mx["dim"], mx["vdim"]
    pos = torch.arange(T) if pos is None else pos
    q = rms_unit((y @ d(W["q"]).T).reshape(T, H, dk), eps) * d(W["q.norm"])
    k = rms_unit((y @ d(W["k"]).T).reshape(T, G, dk), eps) * d(W["k.norm"])
    v = rms_unit((y @ d(W["v"]).T).reshape(T, G, dv), eps)
    rot = mx.get("rot")
    if rot:
        q, k = rotate_half(q, pos, rot), rotate_half(k, pos, rot)
    i, j = pos[:, None], pos[None, :]
    size = (mx.get("mask") or {}).get("size", 0)
    visible = (j <= i) & ((i - j < size) if size else torch.ones_like(i, dtype=torch.bool))
    out = torch.zeros(T, H, dv, dtype=F64)
    cap = mx.get("softcap", 0.0)
    for h in range(H):
        g = h // (H // G)
        s = q[:, h] @ k[:, g].T * mx["scale"]
        if cap:
            s = cap * torch.tanh(s / cap)
        s = s.masked_fill(~visible, -math.inf)
        out[:, h] = torch.softmax(s, -1) @ v[:, g]
    return out.reshape(T, H * dv) @ d(W["o"]).T


def mixer_gated_delta(y, W, mx, eps):
    """Gated delta rule with one decay per head: S <- g S; u = beta (v - S^T k); S <- S + k u^T; o = S^T q."""
    T = y.shape[0]
    H, G, dk, dv = mx["heads"], mx["kv_heads"], mx["dim"], mx["vdim"]
    q = silu(causal_conv(y @ d(W["q"]).T, d(W["q.conv"]))).reshape(T, G, dk)
    k = silu(causal_conv(y @ d(W["k"]).T, d(W["k.conv"]))).reshape(T, G, dk)
    v = silu(causal_conv(y @ d(W["v"]).T, d(W["v.conv"]))).reshape(T, H, dv)
    q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + 1e-6) * dk ** -0.5
    k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
    beta = torch.sigmoid(y @ d(W["b"]).T)
    decay = torch.exp(-torch.exp(d(W["A_log"])) * softplus(y @ d(W["a"]).T + d(W["dt_bias"])))
    S = torch.zeros(H, dk, dv, dtype=F64)
    o = torch.zeros(T, H, dv, dtype=F64)
    for t in range(T):
        for h in range(H):
            g = h // (H // G)
            S[h] = decay[t, h] * S[h]
            u = beta[t, h] * (v[t, h] - S[h].T @ k[t, g])
            S[h] = S[h] + torch.outer(k[t, g], u)
            o[t, h] = S[h].T @ q[t, g]
    r = rms_unit(o, eps) * d(W["norm"])
    gate = silu(y @ d(W["g"]).T).reshape(T, H, dv)
    return (r * gate).reshape(T, H * dv) @ d(W["o"]).T


def mixer_parallel(y, W, mx, eps):
    """Two mixers on the same input; each result is RMS-normed over the width with its own weight, the mean of the two is the result."""
    left = mixer_window_attention(y, sub(W, "left."), mx["left"], eps)
    right = mixer_gated_delta(y, sub(W, "right."), mx["right"], eps)
    return 0.5 * (rms_unit(left, eps) * d(W["left.out"]) + rms_unit(right, eps) * d(W["right.out"]))


def feed_forward(y, W):
    return (silu(y @ d(W["gate"]).T) * (y @ d(W["up"]).T)) @ d(W["down"]).T


def sub(W, prefix):
    return {k[len(prefix):]: v for k, v in W.items() if k.startswith(prefix)}


def run_order(config):
    n = len(config["layers"])
    loop = config.get("loop")
    if not loop:
        return list(range(n))
    block = list(range(loop["start"], loop["stop"]))
    return list(range(loop["start"])) + block * loop["times"] + list(range(loop["stop"], n))


def mixer(kind, y, W, mx, eps):
    if kind == "lightning":
        o = mixer_lightning(y, W, mx)[0]
        return lightning_output(o, y, W, eps)
    if kind == "mamba2":
        return mixer_mamba2(y, W, mx, eps)
    if kind == "parallel":
        return mixer_parallel(y, W, mx, eps)
    raise ValueError(kind)


def hyper_step(X, hc, f):
    """One sublayer on several residual streams: read a weighted sum, write the result into a re-mixed set of streams."""
    u = torch.einsum("s,stw->tw", d(hc["in"]), X)
    r = f(u)
    return torch.einsum("sv,stw->vtw", d(hc["mix"]), X) + d(hc["out"])[:, None, None] * r[None]


def forward(config, W, tokens, trace=False):
    """tokens: list of ids of ONE sequence from position 0.  Returns logits [T, vocab] (and the summed streams after every layer run)."""
    eps = config["norm"]["eps"]
    x = d(W["embed"])[torch.as_tensor(tokens)]
    streams = config.get("streams")
    X = torch.stack([x] * streams) if streams else x[None]
    plain = {"in": torch.ones(1), "mix": torch.ones(1, 1), "out": torch.ones(1)}
    after = []
    for i in run_order(config):
        L, Wl = config["layers"][i], sub(W, f"l{i}.")
        f1 = lambda u: mixer(L["type"], layer_norm(u, d(Wl["norm1"]), d(Wl["norm1.b"]), eps), sub(Wl, "mix."), L["mixer"], eps)
        X = hyper_step(X, sub(Wl, "hc1.") if streams else plain, f1)
        if L.get("mlp"):
            f2 = lambda u: feed_forward(layer_norm(u, d(Wl["norm2"]), d(Wl["norm2.b"]), eps), sub(Wl, "mlp."))
            X = hyper_step(X, sub(Wl, "hc2.") if streams else plain, f2)
        after.append(X.sum(0))
    x = layer_norm(X.sum(0), d(W["final.norm"]), d(W["final.norm.b"]), eps)
    logits = x @ d(W["embed"]).T * config.get("logit_scale", 1.0)
    return (logits, torch.stack(after)) if trace else logits


# ---- small configurations for the tests
def dense(ff=48):
    return {"kind": "dense", "ff": ff}


def lightning_layer(heads=2, dim=8, vdim=12, decay=None, mlp=None):
    decay = decay if decay is not None else [0.5 + 0.49 * (h + 1) / heads for h in range(heads)]
    return {"type": "lightning", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "decay": decay}, "mlp": mlp}


def mamba_layer(heads=4, vdim=6, state=10, groups=2, conv=3, norm_groups=3, mlp=None):
    return {"type": "mamba2", "mixer": {"heads": heads, "vdim": vdim, "state": state, "groups": groups, "conv": conv, "norm_groups": norm_groups},
            "mlp": mlp}


def pair_layer(heads=4, kv_heads=2, dim=16, vdim=12, window=30, rot_dims=8, base=100.0, scaling=True, scale=0.3, softcap=6.0, r_heads=4,
               r_kv_heads=2, r_dim=8, r_vdim=10, conv=3, mlp=None):
    rot = {"base": base, "dims": rot_dims}
    if scaling:   # wavelengths of base 100 over 8 dims: 6, 20, 63, 199: one stays, two are blended, one is slowed down
        rot["scaling"] = scaling if isinstance(scaling, dict) else {"factor": 4.0, "low": 1.0, "high": 8.0, "original": 128}
    left = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "mask": {"size": window}, "rot": rot, "scale": scale, "softcap": softcap}
    right = {"heads": r_heads, "kv_heads": r_kv_heads, "dim": r_dim, "vdim": r_vdim, "conv": conv}
    return {"type": "parallel", "mixer": {"left": left, "right": right}, "mlp": mlp}


def make_config(layers, width=32, vocab=50, streams=3, loop=None, logit_scale=0.5, eps=1e-5):
    import copy

    config = {"architecture": "Silonex", "layers": copy.deepcopy(layers), "norm": {"eps": eps}, "vocab": vocab, "width": width,
              "logit_scale": logit_scale}
    if streams:
        config["streams"] = streams
    if loop:
        config["loop"] = {"start": loop[0], "stop": loop[1], "times": loop[2]}
    return config


def random_model(config, seed=0):
    """Random tensors with the checkpoint's names, rounded to bfloat16 (returned both as float64 for the oracle and packed for the engine)."""
    gen = torch.Generator().manual_seed(seed)
    w = config["width"]
    P = {}

    def lin(name, n_out, n_in, gain=1.0):
        P[name] = gain * torch.randn(n_out, n_in, generator=gen) / math.sqrt(n_in)

    def vec(name, n, mean=0.0, std=0.1):
        P[name] = mean + std * torch.randn(n, generator=gen)

    P["embed"] = torch.randn(config["vocab"], w, generator=gen)
    s = config.get("streams")
    for i, L in enumerate(config["layers"]):
        p, mx, kind = f"l{i}.", L["mixer"], L["type"]
        subs = ["1"] + (["2"] if L.get("mlp") else [])
        for q in subs:
            vec(p + "norm" + q, w, 1.0), vec(p + "norm" + q + ".b", w)
            if s:
                P[p + f"hc{q}.in"] = 1.0 / s + 0.2 * torch.randn(s, generator=gen)
                P[p + f"hc{q}.out"] = 1.0 + 0.2 * torch.randn(s, generator=gen)
                P[p + f"hc{q}.mix"] = torch.eye(s) + 0.15 * torch.randn(s, s, generator=gen)
        pre = p + "mix."
        if kind == "lightning":
            H, dk, dv = mx["heads"], mx["dim"], mx["vdim"]
            lin(pre + "q", H * dk, w), lin(pre + "k", H * dk, w), lin(pre + "v", H * dv, w), lin(pre + "g", H * dv, w), lin(pre + "o", w, H * dv)
            vec(pre + "norm", H * dv, 1.0, 0.2)
        elif kind == "mamba2":
            H, Pd, N, G = mx["heads"], mx["vdim"], mx["state"], mx["groups"]
            inner, ch = H * Pd, H * Pd + 2 * G * N
            lin(pre + "in", 2 * inner + 2 * G * N + H, w)
            P[pre + "conv"] = 0.6 * torch.randn(ch, mx["conv"], generator=gen)
            vec(pre + "conv.b", ch), vec(pre + "dt_bias", H, -0.5, 1.0), vec(pre + "D", H, 1.0, 0.3), vec(pre + "norm", inner, 1.0, 0.2)
            P[pre + "A_log"] = -1.5 + 2.0 * torch.rand(H, generator=gen)
            lin(pre + "o", w, inner)
        elif kind == "parallel":
            a, r = mx["left"], mx["right"]
            H, G, dk, dv = a["heads"], a["kv_heads"], a["dim"], a["vdim"]
            lp = pre + "left."
            lin(lp + "q", H * dk, w, 2.0), lin(lp + "k", G * dk, w, 2.0), lin(lp + "v", G * dv, w), lin(lp + "o", w, H * dv)
            vec(lp + "q.norm", dk, 1.0, 0.2), vec(lp + "k.norm", dk, 1.0, 0.2)
            H, G, dk, dv = r["heads"], r["kv_heads"], r["dim"], r["vdim"]
            rp = pre + "right."
            lin(rp + "q", G * dk, w), lin(rp + "k", G * dk, w), lin(rp + "v", H * dv, w), lin(rp + "b", H, w), lin(rp + "a", H, w, 2.0)
            lin(rp + "g", H * dv, w), lin(rp + "o", w, H * dv)
            for n, c in (("q", G * dk), ("k", G * dk), ("v", H * dv)):
                P[rp + n + ".conv"] = 0.6 * torch.randn(c, r["conv"], generator=gen)
            vec(rp + "dt_bias", H, -1.0, 1.0), vec(rp + "norm", dv, 1.0, 0.2)
            P[rp + "A_log"] = -1.5 + 2.0 * torch.rand(H, generator=gen)
            vec(pre + "left.out", w, 1.0, 0.2), vec(pre + "right.out", w, 1.0, 0.2)
        else:
            raise ValueError(kind)
        if L.get("mlp"):
            ff = L["mlp"]["ff"]
            lin(p + "mlp.gate", ff, w), lin(p + "mlp.up", ff, w), lin(p + "mlp.down", w, ff)
    vec("final.norm", w, 1.0), vec("final.norm.b", w)
    packed = {k: v.to(torch.bfloat16) for k, v in P.items()}
    return {k: v.double() for k, v in packed.items()}, packed


def rel_err(got, want):
    got, want = torch.as_tensor(got, dtype=F64), torch.as_tensor(want, dtype=F64)
    return float((got - want).norm() / want.norm().clamp(min=1e-30))


def greedy(config, W, prompt, n_new):
    """Greedy continuation (ties: the lower id), the whole sequence read anew for every token."""
    toks, out = list(prompt), []
    for _ in range(n_new):
        nxt = int(torch.argmax(forward(config, W, toks)[-1]))
        toks.append(nxt)
        out.append(nxt)
    return out
