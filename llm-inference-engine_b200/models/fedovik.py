"""Fedovik: a decoder-only design whose layers have ONE layer norm (weight and bias) that both sublayers read: x += mixer(ln(x)) + ff(ln(x)).
A block of consecutive layers may run several times with the same weights; every pass has a cache and state of its own and starts with an
entry step x <- W [x ; x0] + step[pass] (x0 the scaled embedding).  Three token mixers --

  * "attention": grouped-query attention with biases on q, k, v and the output, interleaved rotation of the first rot.dims dimensions of
    every head, plain causal mask, weights sigmoid(score + head bias) that are NOT normalised over the keys, a sigmoid output gate;
  * "parallel": two mixers side by side on the same input, result = left_scale * left + right_scale * right --
      left: grouped-query softmax attention over a sliding window, per-head RMS norm of q and k (one weight shared by the heads), no
      rotation, the score lowered by r1 * ln(1 + r2 * distance);
      right: a gated delta rule (short causal convolutions + silu on q, k, v; unit q and k; a decay per head and key channel from a
      low-rank projection; a step size per head; per-head RMS norm of the read-out with a low-rank sigmoid gate);
  * "mlstm": matrix memory with exponential gating, soft-capped log gates and a running maximum that starts at 0 --

beside a gated dense feed-forward W_down (relu(W_gate y) * W_up y), a final layer norm and logits through the embedding table itself.

config.json gives every size; this module turns it plus the checkpoint's tensors into the layer list of hybrid.HybridDecoder.  Every
projection that reads the layer's normed input is a block of rows of ONE matrix (mixer, second mixer, feed-forward gate and up), every
projection that writes the residual a block of columns of ONE matrix, so a layer is two matrix products around its mixers."""
import importlib
import os

from . import register


def _pkg(sub=None):
    base = __package__.rsplit(".", 1)[0]
    return importlib.import_module(base + ("." + sub if sub else ""))


def _attention_spec(m, mx, softmax_window):
    rot = mx.get("rot") or {}
    mask = mx.get("mask") or {}
    return dict(mixer=m.MIXER_ATTN_SCORED, heads=int(mx["heads"]), kv_heads=int(mx.get("kv_heads", mx["heads"])), dim=int(mx["dim"]),
                vdim=int(mx.get("vdim", mx["dim"])), scale=float(mx["scale"]), window=int(mask.get("size", 0)), rot_dims=int(rot.get("dims", 0)),
                rot_base=float(rot.get("base", 10000.0)), attn_weight=m.ATTN_SOFTMAX if softmax_window else m.ATTN_SIGMOID,
                out_gate=0 if softmax_window else 1)


def _delta_spec(m, mx):
    return dict(mixer=m.MIXER_DELTA, heads=int(mx["heads"]), kv_heads=int(mx.get("kv_heads", mx["heads"])), dim=int(mx["dim"]), vdim=int(mx["vdim"]),
                conv=int(mx["conv"]))


def layer_specs(config):
    """The integer / float side of every layer, straight from config.json (no tensors yet)."""
    m = _pkg()
    out = []
    for i, layer in enumerate(config["layers"]):
        mx, kind = layer["mixer"], layer["type"]
        if kind == "attention":
            spec = _attention_spec(m, mx, False)
        elif kind == "parallel":
            spec = _attention_spec(m, mx["left"], True)
            spec.update(side=_delta_spec(m, mx["right"]), mix_scale=float(mx.get("left_scale", 1.0)), side_scale=float(mx.get("right_scale", 1.0)))
        elif kind == "mlstm":
            spec = dict(mixer=m.MIXER_MLSTM, heads=int(mx["heads"]), kv_heads=int(mx["heads"]), dim=int(mx["dim"]), vdim=int(mx["vdim"]),
                        gate_cap=float(mx.get("gate_cap", 0.0)))
        else:
            raise ValueError(f"layer {i}: unknown mixer type {kind!r}")
        spec["norm"] = m.NORM_LN_PARALLEL
        mlp = layer.get("mlp")
        if mlp is None:
            spec.update(mlp=m.MLP_NONE)
        elif mlp.get("kind") == "dense":
            spec.update(mlp=m.MLP_DENSE, expert_ff=int(mlp["ff"]), act=m.ACT_RELU, gated=1)
        else:
            raise ValueError(f"layer {i}: unknown feed-forward kind {mlp.get('kind')!r}")
        out.append(spec)
    return out


def pack_ln(get, name, device):
    """(w, b) of one layer norm as the fp32 vector [w | b] the engine reads."""
    import torch

    return torch.cat([get(name).float().reshape(-1), get(name + ".b").float().reshape(-1)]).to(device).contiguous()


def fuse_layer(spec, get, width, dtype, device):
    """Adds the device tensors of one layer to its spec.  get(name) -> CPU tensor of the checkpoint ('mix.q', 'mlp.up', ...)."""
    import torch

    m = _pkg()

    def vec(name):
        return get(name).to(device=device, dtype=torch.float32).reshape(-1).contiguous()

    def zeros(name):
        return torch.zeros(get(name).shape[0])

    rows, cols = [], []  # blocks of the one input matrix and of the one output matrix

    def attention(sp, pre, biased_out):
        names = [pre + "q", pre + "k", pre + "v"] + ([pre + "g"] if sp["out_gate"] else [])
        rows.extend(get(n) for n in names)
        cols.append(get(pre + "o"))
        bias = [get(n + ".b").float() for n in names[:3]] + ([zeros(pre + "g")] if sp["out_gate"] else [])
        sp["b_in"] = torch.cat(bias).to(device).contiguous()
        if sp["attn_weight"] == m.ATTN_SIGMOID:
            sp["head_bias"] = vec(pre + "pb")
        else:
            sp.update(q_norm=vec(pre + "q.norm"), k_norm=vec(pre + "k.norm"), dist_r1=vec(pre + "r1"), dist_r2=vec(pre + "r2"))
        return get(pre + "o.b").float() if biased_out else None

    def delta(sp, pre):
        rows.extend(get(pre + n) for n in ("q", "k", "v", "b", "a1", "g1"))
        cols.append(get(pre + "o"))
        sp.update(conv_w=torch.cat([get(pre + n + ".conv").float() for n in ("q", "k", "v")], 0).to(device).contiguous(),
                  w_decay=get(pre + "a2").to(device=device, dtype=dtype).contiguous(), decay_bias=vec(pre + "dt_bias"), a_log=vec(pre + "A_log"),
                  w_gate2=get(pre + "g2").to(device=device, dtype=dtype).contiguous(), out_norm=vec(pre + "norm"),
                  decay_rank=int(get(pre + "a1").shape[0]), gate_rank=int(get(pre + "g1").shape[0]))

    b_out = None
    if spec["mixer"] == m.MIXER_ATTN_SCORED and "side" not in spec:
        b_out = attention(spec, "mix.", True)
    elif spec["mixer"] == m.MIXER_ATTN_SCORED:
        attention(spec, "mix.left.", False)
        delta(spec["side"], "mix.right.")
    else:
        names = ("q", "k", "v", "g", "i", "f")
        rows.extend(get("mix." + n) for n in names)
        cols.append(get("mix.o"))
        spec["b_in"] = torch.cat([zeros("mix." + n) for n in names[:4]] + [get("mix.i.b").float(), get("mix.f.b").float()]).to(device).contiguous()
        spec["out_norm"] = vec("mix.norm")
    if spec["mlp"] == m.MLP_DENSE:
        rows.extend([get("mlp.gate"), get("mlp.up")])
        cols.append(get("mlp.down"))
    spec.update(w_in=torch.cat(rows, 0).to(device=device, dtype=dtype).contiguous(), w_out=torch.cat(cols, 1).to(device=device, dtype=dtype).contiguous(),
                pre1=pack_ln(get, "norm1", device))
    if b_out is not None:
        spec["b_out"] = b_out.to(device).contiguous()
    return spec


@register("Fedovik")
class FedovikModel:
    """config + tensors -> a HybridDecoder.  `tensors`: name -> CPU tensor with the checkpoint's names ('embed', 'loop.in', 'l0.mix.q', ...)."""

    def __init__(self, config, tensors, dtype="bfloat16", device="cuda:0", max_tokens=2048, max_seqs=4, max_pages_per_seq=None):
        import torch

        m = _pkg()
        tdt = {"bfloat16": torch.bfloat16, "float16": torch.float16, "float32": torch.float32}[dtype] if isinstance(dtype, str) else dtype
        self.config, self.width, self.vocab = config, int(config["width"]), int(config["vocab"])
        self.eps = float(config["norm"]["eps"])
        specs = layer_specs(config)
        for i, spec in enumerate(specs):
            fuse_layer(spec, lambda n, i=i: tensors[f"l{i}.{n}"], self.width, tdt, device)
        loop = config.get("loop")
        if loop:
            loop = dict(start=int(loop["start"]), stop=int(loop["stop"]), times=int(loop["times"]),
                        w_entry=tensors["loop.in"].to(device=device, dtype=tdt).contiguous(),
                        step=tensors["loop.step"].to(device=device, dtype=torch.float32).contiguous())
        if max_pages_per_seq is None:
            max_pages_per_seq = (max_tokens + m.KV_PAGE_SIZE - 1) // m.KV_PAGE_SIZE
        table = tensors["embed"].to(device=device, dtype=tdt).contiguous()  # the logits come through the embedding table itself
        self.engine = _pkg("hybrid").HybridDecoder(
            self.width, self.vocab, self.eps, specs, table, pack_ln(lambda n: tensors[n], "final.norm", device), table, tdt, device, max_tokens,
            max_seqs, max_pages_per_seq, embed_scale=float((config.get("embedding") or {}).get("scale", 1.0)), final_norm_kind=m.NORM_LN_PARALLEL,
            loop=loop)

    @classmethod
    def from_pretrained(cls, model_dir, config, dtype="bfloat16", device="cuda:0", **limits):
        tensors = _pkg("weights").read_safetensors(os.path.join(model_dir, "model.safetensors"))
        return cls(config, tensors, dtype=dtype, device=device, **limits)
