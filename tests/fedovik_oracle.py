"""A plain float64 restatement of the Fedovik design, one function per mechanism, token by token where the design is recurrent.  It shares
no code with the package: the tests build small random models, run them here and through the engine, and compare.

A model is (config, tensors): config as in config.json, tensors a dict name -> torch tensor with the checkpoint's names.

Notation: x residual stream [T, width]; y the normed input of a layer's sublayers; p the position of a token in its sequence."""
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


def rotate_interleaved(v, pos, dims, base):
    """v [T, heads, dim]: the first `dims` channels rotate in pairs (2i, 2i+1) by the angle pos * base^(-2i/dims)."""
    out = v.clone()
    i = torch.arange(dims // 2, dtype=F64)
    ang = pos.to(F64)[:, None] * base ** (-2.0 * i / dims)          # [T, dims/2]
    c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    a, b = v[..., 0:dims:2], v[..., 1:dims:2]
    out[..., 0:dims:2] = a * c - b * s
    out[..., 1:dims:2] = b * c + a * s
    return out


def mixer_sigmoid_attention(y, W, mx):
    """Rotated grouped-query attention whose weights are sigmoid(score + head bias), not normalised; gated; causal."""
    T = y.shape[0]
    H, G, dk, dv = mx["heads"], mx["kv_heads"], mx["dim"], mx["vdim"]
    q = (y @ d(W["q"]).T + d(W["q.b"])).reshape(T, H, dk)
    k = (y @ d(W["k"]).T + d(W["k.b"])).reshape(T, G, dk)
    v = (y @ d(W["v"]).T + d(W["v.b"])).reshape(T, G, dv)
    pos = torch.arange(T)
    rot = mx.get("rot")
    if rot:
        q = rotate_interleaved(q, pos, rot["dims"], rot["base"])
        k = rotate_interleaved(k, pos, rot["dims"], rot["base"])
    out = torch.zeros(T, H, dv, dtype=F64)
    for h in range(H):
        g = h // (H // G)
        s = q[:, h] @ k[:, g].T * mx["scale"] + d(W["pb"])[h]
        w = torch.sigmoid(s) * torch.tril(torch.ones(T, T, dtype=F64))
        out[:, h] = w @ v[:, g]
    gate = torch.sigmoid(y @ d(W["g"]).T)
    return (out.reshape(T, H * dv) * gate) @ d(W["o"]).T + d(W["o.b"])


def mixer_window_attention(y, W, mx, eps):
    """Grouped-query softmax attention over a sliding window, per-head RMS norm of q and k, no rotation, a logarithmic distance penalty."""
    T = y.shape[0]
    H, G, dk, dv = mx["heads"], mx["kv_heads"], mx["dim"], mx["vdim"]
    q = (y @ d(W["q"]).T + d(W["q.b"])).reshape(T, H, dk)
    k = (y @ d(W["k"]).T + d(W["k.b"])).reshape(T, G, dk)
    v = (y @ d(W["v"]).T + d(W["v.b"])).reshape(T, G, dv)
    q = rms_unit(q, eps) * d(W["q.norm"])
    k = rms_unit(k, eps) * d(W["k.norm"])
    win = mx["mask"]["size"]
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    dist = (i - j).to(F64)
    seen = (i - j >= 0) & (i - j < win)
    out = torch.zeros(T, H, dv, dtype=F64)
    for h in range(H):
        g = h // (H // G)
        s = q[:, h] @ k[:, g].T * mx["scale"]
        s = s - d(W["r1"])[h] * torch.log1p(d(W["r2"])[h] * dist.clamp(min=0))
        s = s.masked_fill(~seen, -math.inf)
        out[:, h] = torch.softmax(s, -1) @ v[:, g]
    return out.reshape(T, H * dv) @ d(W["o"]).T


def short_conv_silu(z, taps):
    """z [T, C], taps [C, n]: causal per-channel convolution (the last tap meets the current token, zeros before the start), then silu."""
    T, C = z.shape
    n = taps.shape[1]
    padded = torch.cat([torch.zeros(n - 1, C, dtype=F64), z], 0)
    out = torch.zeros(T, C, dtype=F64)
    for j in range(n):
        out += padded[j:j + T] * taps[:, j]
    return out * torch.sigmoid(out)


def mixer_gated_delta(y, W, mx, eps):
    """Gated delta rule with a decay per head and key channel, token by token."""
    T = y.shape[0]
    H, G, dk, dv = mx["heads"], mx["kv_heads"], mx["dim"], mx["vdim"]
    q = short_conv_silu(y @ d(W["q"]).T, d(W["q.conv"])).reshape(T, G, dk)
    k = short_conv_silu(y @ d(W["k"]).T, d(W["k.conv"])).reshape(T, G, dk)
    v = short_conv_silu(y @ d(W["v"]).T, d(W["v.conv"])).reshape(T, H, dv)
    q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + 1e-6) * dk ** -0.5
    k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
    beta = torch.sigmoid(y @ d(W["b"]).T)                                            # [T, H]
    dt = torch.nn.functional.softplus((y @ d(W["a1"]).T) @ d(W["a2"]).T + d(W["dt_bias"])).reshape(T, H, dk)
    decay = torch.exp(-torch.exp(d(W["A_log"]))[None, :, None] * dt)                 # [T, H, dk]
    gate = torch.sigmoid((y @ d(W["g1"]).T) @ d(W["g2"]).T).reshape(T, H, dv)
    S = torch.zeros(H, dk, dv, dtype=F64)
    o = torch.zeros(T, H, dv, dtype=F64)
    for t in range(T):
        for h in range(H):
            g = h // (H // G)
            S[h] = decay[t, h][:, None] * S[h]
            u = beta[t, h] * (v[t, h] - S[h].T @ k[t, g])
            S[h] = S[h] + torch.outer(k[t, g], u)
            o[t, h] = S[h].T @ q[t, g]
    o = rms_unit(o, eps) * d(W["norm"]) * gate
    return o.reshape(T, H * dv) @ d(W["o"]).T


def mixer_pair(y, W, mx, eps):
    left = mixer_window_attention(y, {k[5:]: v for k, v in W.items() if k.startswith("left.")}, mx["left"], eps)
    right = mixer_gated_delta(y, {k[6:]: v for k, v in W.items() if k.startswith("right.")}, mx["right"], eps)
    return mx["left_scale"] * left + mx["right_scale"] * right


def mixer_mlstm(y, W, mx, eps):
    """Matrix memory with exponential gating and a running maximum that starts at 0."""
    T = y.shape[0]
    H, dk, dv, cap = mx["heads"], mx["dim"], mx["vdim"], mx["gate_cap"]
    q = (y @ d(W["q"]).T).reshape(T, H, dk) * dk ** -0.5
    k = (y @ d(W["k"]).T).reshape(T, H, dk)
    v = (y @ d(W["v"]).T).reshape(T, H, dv)
    gi = cap * torch.tanh((y @ d(W["i"]).T + d(W["i.b"])) / cap)
    gf = torch.nn.functional.logsigmoid(cap * torch.tanh((y @ d(W["f"]).T + d(W["f.b"])) / cap))
    S = torch.zeros(H, dk, dv, dtype=F64)
    n = torch.zeros(H, dk, dtype=F64)
    m = torch.zeros(H, dtype=F64)
    o = torch.zeros(T, H, dv, dtype=F64)
    for t in range(T):
        for h in range(H):
            m_new = torch.maximum(gf[t, h] + m[h], gi[t, h])
            a, b = torch.exp(gf[t, h] + m[h] - m_new), torch.exp(gi[t, h] - m_new)
            S[h] = a * S[h] + b * torch.outer(k[t, h], v[t, h])
            n[h] = a * n[h] + b * k[t, h]
            m[h] = m_new
            den = torch.maximum((n[h] @ q[t, h]).abs(), torch.exp(-m_new)) + 1e-6
            o[t, h] = S[h].T @ q[t, h] / den
    o = rms_unit(o, eps).reshape(T, H * dv) * d(W["norm"]) * torch.sigmoid(y @ d(W["g"]).T)
    return o @ d(W["o"]).T


def feed_forward(y, W):
    return (torch.relu(y @ d(W["gate"]).T) * (y @ d(W["up"]).T)) @ d(W["down"]).T


def layer_order(config):
    """Layer indices in the order they run, with (pass number, first of its pass) for the looped block's entry steps."""
    n = len(config["layers"])
    loop = config.get("loop")
    if not loop:
        return [(i, None) for i in range(n)]
    runs = [(i, None) for i in range(loop["start"])]
    for t in range(loop["times"]):
        runs += [(i, t if i == loop["start"] else None) for i in range(loop["start"], loop["stop"])]
    return runs + [(i, None) for i in range(loop["stop"], n)]


def forward(config, tensors, tokens, trace=False):
    """Logits [T, vocab] of one sequence read from position 0 (and the residual stream after every layer run)."""
    eps = config["norm"]["eps"]
    emb = d(tensors["embed"])
    x = emb[torch.as_tensor(tokens, dtype=torch.long)] * config["embedding"]["scale"]
    x0 = x.clone()
    seen = []
    for li, entry in layer_order(config):
        L = config["layers"][li]
        W = {k[len(f"l{li}."):]: v for k, v in tensors.items() if k.startswith(f"l{li}.")}
        if entry is not None:
            x = torch.cat([x, x0], -1) @ d(tensors["loop.in"]).T + d(tensors["loop.step"])[entry]
        y = layer_norm(x, d(W["norm1"]), d(W["norm1.b"]), eps)
        mw = {k[4:]: v for k, v in W.items() if k.startswith("mix.")}
        if L["type"] == "attention":
            r = mixer_sigmoid_attention(y, mw, L["mixer"])
        elif L["type"] == "parallel":
            r = mixer_pair(y, mw, L["mixer"], eps)
        elif L["type"] == "mlstm":
            r = mixer_mlstm(y, mw, L["mixer"], eps)
        else:
            raise ValueError(L["type"])
        if L.get("mlp"):
            r = r + feed_forward(y, {k[4:]: v for k, v in W.items() if k.startswith("mlp.")})
        x = x + r
        seen.append(x.clone())
    logits = layer_norm(x, d(tensors["final.norm"]), d(tensors["final.norm.b"]), eps) @ emb.T
    return (logits, torch.stack(seen)) if trace else logits


# ------------------------------------------------------------------ small random models for the tests
def attention_layer(heads=4, kv_heads=2, dim=16, vdim=8, rot_dims=None, base=10000.0, scale=None, mlp=None):
    rot_dims = dim if rot_dims is None else rot_dims
    mx = dict(heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim, scale=dim ** -0.5 if scale is None else scale)
    if rot_dims:
        mx["rot"] = dict(base=base, dims=rot_dims)
    return dict(type="attention", mixer=mx, mlp=mlp)


def pair_layer(heads=4, kv_heads=2, dim=16, vdim=24, window=24, scale=None, left_scale=0.7, right_scale=1.1, r_heads=2, r_kv_heads=1, r_dim=8,
               r_vdim=16, conv=4, mlp=None):
    left = dict(heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim, scale=dim ** -0.5 if scale is None else scale, mask=dict(size=window))
    right = dict(heads=r_heads, kv_heads=r_kv_heads, dim=r_dim, vdim=r_vdim, conv=conv)
    return dict(type="parallel", mixer=dict(left=left, right=right, left_scale=left_scale, right_scale=right_scale), mlp=mlp)


def mlstm_layer(heads=2, dim=12, vdim=16, gate_cap=8.0, mlp=None):
    return dict(type="mlstm", mixer=dict(heads=heads, dim=dim, vdim=vdim, gate_cap=gate_cap), mlp=mlp)


def dense(ff=40):
    return dict(kind="dense", ff=ff)


def make_config(layers, width=32, vocab=50, embed_scale=2.0, loop=None, eps=1e-5):
    config = dict(architecture="Fedovik", width=width, vocab=vocab, embedding=dict(scale=embed_scale), norm=dict(eps=eps), layers=layers)
    if loop:
        config["loop"] = dict(start=loop[0], stop=loop[1], times=loop[2])
    return config


def make_weights(config, seed=0, low_rank=6):
    """Random weights whose values are exact in bfloat16: (float64 dict for this file, bfloat16 dict as a checkpoint holds them)."""
    gen = torch.Generator().manual_seed(seed)
    w = config["width"]
    P = {}

    def lin(name, out, inp, gain=1.0):
        P[name] = torch.randn(out, inp, generator=gen) * gain / math.sqrt(inp)

    def vec(name, n, mean=0.0, std=0.1):
        P[name] = mean + std * torch.randn(n, generator=gen)

    P["embed"] = torch.randn(config["vocab"], w, generator=gen)
    if config.get("loop"):
        P["loop.in"] = torch.cat([torch.eye(w), 0.3 * torch.eye(w)], 1) + 0.3 * torch.randn(w, 2 * w, generator=gen) / math.sqrt(w)
        vec("loop.step", config["loop"]["times"] * w)
        P["loop.step"] = P["loop.step"].view(config["loop"]["times"], w)
    for i, L in enumerate(config["layers"]):
        p, mx = f"l{i}.", L["mixer"]
        vec(p + "norm1", w, 1.0), vec(p + "norm1.b", w)

        def attention(pre, a, sigmoid):
            H, G, dk, dv = a["heads"], a["kv_heads"], a["dim"], a["vdim"]
            lin(pre + "q", H * dk, w, 2.0), lin(pre + "k", G * dk, w, 2.0), lin(pre + "v", G * dv, w), lin(pre + "o", w, H * dv)
            vec(pre + "q.b", H * dk, 0.0, 0.3), vec(pre + "k.b", G * dk, 0.0, 0.3), vec(pre + "v.b", G * dv)
            if sigmoid:
                lin(pre + "g", H * dv, w), vec(pre + "o.b", w), vec(pre + "pb", H, -2.0, 0.5)
            else:
                vec(pre + "q.norm", dk, 1.0, 0.2), vec(pre + "k.norm", dk, 1.0, 0.2)
                P[pre + "r1"] = 0.2 + torch.rand(H, generator=gen)
                P[pre + "r2"] = 0.5 + torch.rand(H, generator=gen)

        if L["type"] == "attention":
            attention(p + "mix.", mx, True)
        elif L["type"] == "parallel":
            attention(p + "mix.left.", mx["left"], False)
            r, pre = mx["right"], p + "mix.right."
            H, G, dk, dv = r["heads"], r["kv_heads"], r["dim"], r["vdim"]
            lin(pre + "q", G * dk, w), lin(pre + "k", G * dk, w), lin(pre + "v", H * dv, w), lin(pre + "b", H, w), lin(pre + "o", w, H * dv)
            for n, c in (("q", G * dk), ("k", G * dk), ("v", H * dv)):
                P[pre + n + ".conv"] = 0.6 * torch.randn(c, r["conv"], generator=gen)
            lin(pre + "a1", low_rank, w), lin(pre + "a2", H * dk, low_rank, 2.0), vec(pre + "dt_bias", H * dk, -1.0, 1.0)
            P[pre + "A_log"] = -1.5 + 2.0 * torch.rand(H, generator=gen)
            lin(pre + "g1", low_rank + 1, w), lin(pre + "g2", H * dv, low_rank + 1, 2.0), vec(pre + "norm", dv, 1.0, 0.2)
        else:
            H, dk, dv = mx["heads"], mx["dim"], mx["vdim"]
            pre = p + "mix."
            lin(pre + "q", H * dk, w), lin(pre + "k", H * dk, w), lin(pre + "v", H * dv, w), lin(pre + "g", H * dv, w), lin(pre + "o", w, H * dv)
            lin(pre + "i", H, w, 3.0), lin(pre + "f", H, w, 3.0), vec(pre + "i.b", H, 0.0, 1.0), vec(pre + "f.b", H, 2.0, 1.0)
            vec(pre + "norm", H * dv, 1.0, 0.2)
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
