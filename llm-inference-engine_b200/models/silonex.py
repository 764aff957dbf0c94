"""Silonex: a decoder-only design of pre-norm layers on several residual streams.  A sublayer reads a weighted sum of the streams through a
layer norm (weight and bias), and its result rewrites all streams at once: x_t <- sum_s mix[s][t] x_s + out[t] * result; the model's
result is the sum of the streams.  A block of consecutive layers may run several times with the same weights, every pass with a cache
and state of its own and nothing else between the passes.  Three token mixers --

  * "lightning": linear attention with one constant decay per head (q, k, v = silu of their projections; fp32 matrix state per head), RMS
    norm over the concatenated heads, sigmoid output gate;
  * "mamba2": a state-space mixer -- one input projection z | x | B | C | dt, a short causal convolution with bias and silu on x | B | C, a
    step size dt = softplus(dt + bias) per head, S <- exp(-exp(A_log) dt) S + dt B x^T, out = S^T C + D x, gated by silu(z), RMS-normed in
    equal groups;
  * "parallel": two mixers side by side on the same input; each one's projected result is RMS-normed over the width with a weight of its own
    and the mean of the two is the sublayer's result --
      left: grouped-query softmax attention over a sliding window, per-head RMS norm of q and k (one weight shared by the heads), rotation in
      halves (i, i + dims/2) with the long wavelengths slowed down, values cached divided by their root mean square, scores capped by tanh;
      right: a gated delta rule (short causal convolutions + silu on q, k, v; unit q and k; one decay and one step size per head; per-head
      RMS norm of the read-out with a silu gate);

beside a gated dense feed-forward W_down (silu(W_gate y) * W_up y), a final layer norm and logits through the embedding table itself, times
logit_scale.

config.json gives every size and constant; this module turns it plus the checkpoint's tensors into the layer list of hybrid.HybridDecoder."""
import importlib
import os

from . import register


def _pkg(sub=None):
    base = __package__.rsplit(".", 1)[0]
    return importlib.import_module(base + ("." + sub if sub else ""))


def _num(d, key, default, kind=float):
    """d[key] as a number; a key that is absent or null takes the default (the mechanism is switched off)."""
    v = d.get(key)
    return kind(default if v is None else v)


def _attention_spec(m, mx):
    rot = mx.get("rot") or {}
    sc = rot.get("scaling") or {}
    mask = mx.get("mask") or {}
    heads = int(mx["heads"])
    dim = int(mx["dim"])
    return dict(mixer=m.MIXER_ATTN_SCORED, heads=heads, kv_heads=_num(mx, "kv_heads", heads, int), dim=dim, vdim=_num(mx, "vdim", dim, int),
                scale=float(mx["scale"]), softcap=_num(mx, "softcap", 0.0), window=_num(mask, "size", 0, int), rot_dims=_num(rot, "dims", 0, int),
                rot_base=_num(rot, "base", 10000.0), rot_half=1, rot_factor=_num(sc, "factor", 0.0), rot_low=_num(sc, "low", 0.0),
                rot_high=_num(sc, "high", 0.0), rot_original=_num(sc, "original", 0.0), v_norm=1, attn_weight=m.ATTN_SOFTMAX, out_gate=0)


def _delta_spec(m, mx):
    return dict(mixer=m.MIXER_DELTA, heads=int(mx["heads"]), kv_heads=_num(mx, "kv_heads", mx["heads"], int), dim=int(mx["dim"]), vdim=int(mx["vdim"]),
                conv=int(mx["conv"]), decay_rank=0, gate_rank=0, gate_act=1)


def layer_specs(config):
    """The integer / float side of every layer, straight from config.json (no tensors yet)."""
    m = _pkg()
    out = []
    for i, layer in enumerate(config["layers"]):
        mx, kind = layer["mixer"], layer["type"]
        if kind == "lightning":
            spec = dict(mixer=m.MIXER_LINEAR, heads=int(mx["heads"]), kv_heads=int(mx["heads"]), dim=int(mx["dim"]), vdim=int(mx["vdim"]),
                        decay=[float(v) for v in mx["decay"]])
            if len(spec["decay"]) != spec["heads"]:
                raise ValueError(f"layer {i}: {len(spec['decay'])} decays for {spec['heads']} heads")
        elif kind == "mamba2":
            spec = dict(mixer=m.MIXER_SSD, heads=int(mx["heads"]), kv_heads=_num(mx, "groups", 1, int), dim=int(mx["state"]), vdim=int(mx["vdim"]),
                        conv=int(mx["conv"]), norm_groups=_num(mx, "norm_groups", 1, int))
        elif kind == "parallel":
            spec = _attention_spec(m, mx["left"])
            spec.update(side=_delta_spec(m, mx["right"]), mix_scale=0.5, side_scale=0.5)
        else:
            raise ValueError(f"layer {i}: unknown mixer type {kind!r}")
        spec["norm"] = m.NORM_LN_PRE
        mlp = layer.get("mlp")
        if mlp is None:
            spec.update(mlp=m.MLP_NONE)
        elif mlp.get("kind") == "dense":
            spec.update(mlp=m.MLP_DENSE, expert_ff=int(mlp["ff"]), act=m.ACT_SILU, gated=1)
        else:
            raise ValueError(f"layer {i}: unknown feed-forward kind {mlp.get('kind')!r}")
        out.append(spec)
    return out


def pack_ln(get, name, device):
    """(w, b) of one layer norm as the fp32 vector [w | b] the engine reads."""
    import torch

    return torch.cat([get(name).float().reshape(-1), get(name + ".b").float().reshape(-1)]).to(device).contiguous()


def pack_streams(get, name, streams, device):
    """The coefficients of one sublayer's step on the residual streams as the fp32 vector [in | out | mix (from, to)]."""
    import torch

    parts = [get(name + ".in").float().reshape(-1), get(name + ".out").float().reshape(-1), get(name + ".mix").float().reshape(-1)]
    if parts[0].numel() != streams or parts[1].numel() != streams or parts[2].numel() != streams * streams:
        raise ValueError(f"{name}: coefficients do not fit {streams} streams")
    return torch.cat(parts).to(device).contiguous()


def fuse_layer(spec, get, streams, dtype, device):
    """Adds the device tensors of one layer to its spec.  get(name) -> CPU tensor of the checkpoint ('mix.q', 'mlp.up', ...)."""
    import torch

    m = _pkg()

    def vec(name):
        return get(name).to(device=device, dtype=torch.float32).reshape(-1).contiguous()

    def mat(*names):
        return torch.cat([get(n) for n in names], 0).to(device=device, dtype=dtype).contiguous()

    rows = []
    if spec["mixer"] == m.MIXER_LINEAR:
        rows += ["mix.q", "mix.k", "mix.v", "mix.g"]
        spec.update(w_out=mat("mix.o"), out_norm=vec("mix.norm"), head_decay=torch.tensor(spec.pop("decay"), dtype=torch.float32, device=device))
    elif spec["mixer"] == m.MIXER_SSD:
        rows += ["mix.in"]
        spec.update(w_out=mat("mix.o"), out_norm=vec("mix.norm"), conv_w=get("mix.conv").float().to(device).contiguous(), conv_b=vec("mix.conv.b"),
                    decay_bias=vec("mix.dt_bias"), a_log=vec("mix.A_log"), skip=vec("mix.D"))
        if tuple(spec["conv_w"].shape) != (spec["heads"] * spec["vdim"] + 2 * spec["kv_heads"] * spec["dim"], spec["conv"]):
            raise ValueError("mix.conv: shape does not fit the mixer's channels and taps")
    else:
        side = spec["side"]
        rows += ["mix.left.q", "mix.left.k", "mix.left.v"] + ["mix.right." + n for n in ("q", "k", "v", "b", "a", "g")]
        spec.update(w_out=mat("mix.left.o"), q_norm=vec("mix.left.q.norm"), k_norm=vec("mix.left.k.norm"), branch_norm=vec("mix.left.out"))
        side.update(w_out=mat("mix.right.o"), conv_w=torch.cat([get("mix.right." + n + ".conv").float() for n in ("q", "k", "v")], 0).to(device).contiguous(),
                    decay_bias=vec("mix.right.dt_bias"), a_log=vec("mix.right.A_log"), out_norm=vec("mix.right.norm"), branch_norm=vec("mix.right.out"))
    spec.update(w_in=mat(*rows), pre1=pack_ln(get, "norm1", device))
    if streams:
        spec["hc1"] = pack_streams(get, "hc1", streams, device)
    if spec["mlp"] == m.MLP_DENSE:
        spec.update(w_up=mat("mlp.gate", "mlp.up"), w_down=mat("mlp.down"), pre2=pack_ln(get, "norm2", device))
        if streams:
            spec["hc2"] = pack_streams(get, "hc2", streams, device)
    return spec


@register("Silonex")
class SilonexModel:
    """config + tensors -> a HybridDecoder.  `tensors`: name -> CPU tensor with the checkpoint's names ('embed', 'l0.mix.q', ...)."""

    def __init__(self, config, tensors, dtype="bfloat16", device="cuda:0", max_tokens=2048, max_seqs=4, max_pages_per_seq=None):
        import torch

        m = _pkg()
        tdt = {"bfloat16": torch.bfloat16, "float16": torch.float16, "float32": torch.float32}[dtype] if isinstance(dtype, str) else dtype
        self.config, self.width, self.vocab = config, int(config["width"]), int(config["vocab"])
        self.eps = float(config["norm"]["eps"])
        streams = int(config.get("streams") or 0)  # absent: the plain residual sum
        specs = layer_specs(config)
        for i, spec in enumerate(specs):
            fuse_layer(spec, lambda n, i=i: tensors[f"l{i}.{n}"], streams, tdt, device)
        loop = config.get("loop")
        if loop:
            loop = dict(start=int(loop["start"]), stop=int(loop["stop"]), times=int(loop["times"]))
            if not 0 <= loop["start"] <= loop["stop"] <= len(specs) or loop["times"] < 0:
                raise ValueError(f"loop {loop} does not fit {len(specs)} layers")
            if loop["times"] == 0:  # a block that runs no time at all
                del specs[loop["start"]:loop["stop"]]
            if loop["times"] <= 1 or loop["stop"] == loop["start"]:
                loop = None
        if max_pages_per_seq is None:
            max_pages_per_seq = (max_tokens + m.KV_PAGE_SIZE - 1) // m.KV_PAGE_SIZE
        table = tensors["embed"].to(device=device, dtype=tdt).contiguous()  # the logits come through the embedding table itself
        self.engine = _pkg("hybrid").HybridDecoder(
            self.width, self.vocab, self.eps, specs, table, pack_ln(lambda n: tensors[n], "final.norm", device), table, tdt, device, max_tokens,
            max_seqs, max_pages_per_seq, final_norm_kind=m.NORM_LN_PRE, loop=loop, logit_scale=_num(config, "logit_scale", 1.0), streams=streams)

    @classmethod
    def from_pretrained(cls, model_dir, config, dtype="bfloat16", device="cuda:0", **limits):
        tensors = _pkg("weights").read_safetensors(os.path.join(model_dir, "model.safetensors"))
        return cls(config, tensors, dtype=dtype, device=device, **limits)
