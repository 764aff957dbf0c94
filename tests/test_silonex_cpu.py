"""Host-side checks of the Silonex model class (no GPU): the registry, the configuration reader, and the oracle's own mechanisms."""
import importlib
import math

import pytest
import torch

import silonex_oracle as ref
from util import b200

F64 = torch.float64


def test_registry_names_the_design():
    models = importlib.import_module("llm-inference-engine_b200.models")
    assert "silonex" in models.architectures()
    assert models.architecture_of({"architecture": "Silonex"}) == "Silonex"


def test_layer_specs_follow_the_configuration():
    m = b200()
    f = importlib.import_module("llm-inference-engine_b200.models.silonex")
    config = ref.make_config([ref.lightning_layer(heads=3, dim=10, vdim=7, decay=[0.5, 0.75, 1.0], mlp=ref.dense(13)),
                              ref.mamba_layer(heads=6, vdim=5, state=9, groups=3, conv=2, norm_groups=5),
                              ref.pair_layer(heads=4, kv_heads=1, dim=12, vdim=20, window=11, rot_dims=6, base=77.0, scale=0.3, softcap=4.5, r_heads=6,
                                             r_kv_heads=2, r_dim=5, r_vdim=9, conv=3)])
    a, b, c = f.layer_specs(config)
    assert (a["mixer"], a["norm"], a["heads"], a["dim"], a["vdim"], a["decay"]) == (m.MIXER_LINEAR, m.NORM_LN_PRE, 3, 10, 7, [0.5, 0.75, 1.0])
    assert (a["mlp"], a["expert_ff"], a["act"], a["gated"]) == (m.MLP_DENSE, 13, m.ACT_SILU, 1)
    assert (b["mixer"], b["heads"], b["kv_heads"], b["dim"], b["vdim"], b["conv"], b["norm_groups"], b["mlp"]) == (m.MIXER_SSD, 6, 3, 9, 5, 2, 5, m.MLP_NONE)
    assert (c["mixer"], c["heads"], c["kv_heads"], c["dim"], c["vdim"], c["window"], c["rot_dims"], c["rot_half"], c["v_norm"], c["attn_weight"]) == \
        (m.MIXER_ATTN_SCORED, 4, 1, 12, 20, 11, 6, 1, 1, m.ATTN_SOFTMAX)
    assert c["scale"] == 0.3 and c["softcap"] == 4.5 and c["rot_base"] == 77.0 and c["mix_scale"] == 0.5 and c["side_scale"] == 0.5
    assert (c["rot_factor"], c["rot_low"], c["rot_high"], c["rot_original"]) == (4.0, 1.0, 8.0, 128.0)
    s = c["side"]
    assert (s["mixer"], s["heads"], s["kv_heads"], s["dim"], s["vdim"], s["conv"], s["decay_rank"], s["gate_act"]) == (m.MIXER_DELTA, 6, 2, 5, 9, 3, 0, 1)
    with pytest.raises(ValueError):
        f.layer_specs(ref.make_config([{"type": "conv", "mixer": {"heads": 1, "dim": 4}, "mlp": None}]))
    with pytest.raises(ValueError):
        f.layer_specs(ref.make_config([ref.mamba_layer(mlp={"kind": "moe"})]))
    with pytest.raises(ValueError):
        f.layer_specs(ref.make_config([ref.lightning_layer(heads=2, decay=[0.5])]))


def test_layer_specs_switch_off_what_is_absent_or_null():
    m = b200()
    f = importlib.import_module("llm-inference-engine_b200.models.silonex")
    pair = ref.pair_layer(heads=6, kv_heads=3, dim=10, vdim=14, r_heads=2, r_kv_heads=2, r_dim=6, r_vdim=4, conv=2)
    left, right = pair["mixer"]["left"], pair["mixer"]["right"]
    for absent in (False, True):  # the keys left out, then present with null
        for key in ("mask", "rot", "softcap", "kv_heads", "vdim"):
            if absent:
                left.pop(key, None)
            else:
                left[key] = None
        if absent:
            right.pop("kv_heads", None)
        else:
            right["kv_heads"] = None
        mamba = ref.mamba_layer(heads=4, vdim=6, state=10, groups=2, conv=3, norm_groups=3)
        if absent:
            del mamba["mixer"]["norm_groups"], mamba["mixer"]["groups"]
        else:
            mamba["mixer"]["norm_groups"] = mamba["mixer"]["groups"] = None
        c, b = f.layer_specs(ref.make_config([pair, mamba]))
        assert (c["window"], c["rot_dims"], c["softcap"], c["rot_factor"], c["kv_heads"], c["vdim"]) == (0, 0, 0.0, 0.0, 6, 10)
        assert c["side"]["kv_heads"] == 2 and (b["norm_groups"], b["kv_heads"]) == (1, 1)
    left["rot"] = {"dims": 4, "base": 50.0, "scaling": None}  # rotation without slowed wavelengths
    c = f.layer_specs(ref.make_config([pair]))[0]
    assert (c["rot_dims"], c["rot_base"], c["rot_factor"], c["mixer"]) == (4, 50.0, 0.0, m.MIXER_ATTN_SCORED)


def test_oracle_run_order_of_looped_blocks():
    assert ref.run_order(ref.make_config([0] * 4)) == [0, 1, 2, 3]
    assert ref.run_order(ref.make_config([0] * 4, loop=(1, 3, 2))) == [0, 1, 2, 1, 2, 3]
    assert ref.run_order(ref.make_config([0] * 2, loop=(0, 1, 1))) == [0, 1]
    assert ref.run_order(ref.make_config([0] * 3, loop=(1, 2, 0))) == [0, 2]


def test_oracle_rotation_pairs_halves_and_leaves_the_rest():
    v = (torch.arange(12, dtype=F64) + 1).view(2, 1, 6)
    rot = {"dims": 4, "base": 100.0}
    out = ref.rotate_half(v, torch.tensor([0, 3]), rot)
    assert torch.equal(out[0], v[0])                         # position 0 turns nothing
    assert torch.equal(out[1, 0, 4:], v[1, 0, 4:])           # past `dims`: unchanged
    c, s = math.cos(3.0), math.sin(3.0)                      # pair (0, 2) turns by 3 * 100^0
    assert torch.allclose(out[1, 0, 0], v[1, 0, 0] * c - v[1, 0, 2] * s) and torch.allclose(out[1, 0, 2], v[1, 0, 2] * c + v[1, 0, 0] * s)
    c2, s2 = math.cos(0.3), math.sin(0.3)                    # pair (1, 3) by 3 * 100^(-2/4)
    assert torch.allclose(out[1, 0, 1], v[1, 0, 1] * c2 - v[1, 0, 3] * s2)


def test_oracle_slows_long_wavelengths_only():
    rot = {"dims": 8, "base": 100.0, "scaling": {"factor": 4.0, "low": 1.0, "high": 8.0, "original": 128}}
    f, plain = ref.rotary_frequencies(rot), ref.rotary_frequencies({"dims": 8, "base": 100.0})
    assert f[0] == plain[0]                                   # wavelength 2 pi < 128 / 8
    assert torch.allclose(f[3], plain[3] / 4.0)               # wavelength 199 > 128
    wl = 2 * math.pi / float(plain[2])                        # 63: between the two
    s = (128 / wl - 1.0) / 7.0
    assert torch.allclose(f[2], (1 - s) * plain[2] / 4.0 + s * plain[2]) and plain[2] / 4.0 < f[2] < plain[2]


def test_oracle_convolution_is_causal_and_ends_on_the_current_token():
    z = torch.randn(7, 2, dtype=F64)
    taps = torch.tensor([[0.0, 0.0, 1.0], [1.0, 0.0, 0.0]], dtype=F64)
    out = ref.causal_conv(z, taps, torch.tensor([0.0, 0.5], dtype=F64))
    assert torch.allclose(out[:, 0], z[:, 0])                                       # the last tap alone: the token itself
    assert torch.allclose(out[2:, 1], z[:-2, 1] + 0.5) and torch.allclose(out[:2, 1], torch.full((2,), 0.5, dtype=F64))


def test_oracle_streams_mix_from_rows_to_columns():
    X = torch.stack([torch.ones(1, 2, dtype=F64), 10 * torch.ones(1, 2, dtype=F64)])
    hc = {"in": torch.tensor([1.0, 0.0]), "out": torch.tensor([0.0, 1.0]), "mix": torch.tensor([[0.0, 1.0], [0.0, 0.0]])}
    new = ref.hyper_step(X, hc, lambda u: u + 100.0)          # reads stream 0; stream 0 moves to stream 1; the result goes to stream 1
    assert torch.equal(new[0], torch.zeros(1, 2, dtype=F64)) and torch.equal(new[1], torch.full((1, 2), 102.0, dtype=F64))


def test_oracle_delta_rule_writes_before_it_reads():
    """With no decay, a full step and a unit key, the token's own value comes straight back."""
    config = ref.make_config([ref.pair_layer(r_heads=1, r_kv_heads=1, r_dim=4, r_vdim=3, conv=1)])
    W, _ = ref.random_model(config, seed=1)
    mx = config["layers"][0]["mixer"]["right"]
    R = {k: v.clone() for k, v in ref.sub(W, "l0.mix.right.").items()}
    R["A_log"][:] = -60.0                      # decay exp(-tiny) = 1
    R["b"][:] = 1e3                            # beta -> 1 for the positive input below
    R["norm"][:] = 1.0
    R["g"][:] = 0.0                            # silu(0) = 0 would hide everything: use a gate of 1 instead
    R["g"] += 1.2784645 / config["width"]      # silu(1.2784645) = 1
    R["o"] = torch.eye(3, dtype=F64)
    y = torch.ones(1, config["width"], dtype=F64)
    q, k, v = (ref.silu(ref.causal_conv(y @ R[n].T, R[n + ".conv"])) for n in ("q", "k", "v"))
    qn, kn = q / torch.sqrt((q * q).sum() + 1e-6) * 4 ** -0.5, k / torch.sqrt((k * k).sum() + 1e-6)
    o = (kn @ qn.T) * v                        # S = k v^T after one token
    assert torch.allclose(ref.mixer_gated_delta(y, R, mx, 0.0), o / torch.sqrt((o * o).mean()), atol=1e-6)


def test_oracle_state_space_step_of_one_token():
    config = ref.make_config([ref.mamba_layer(heads=1, vdim=2, state=3, groups=1, conv=1, norm_groups=1)])
    W, _ = ref.random_model(config, seed=2)
    M = {k: v.clone() for k, v in ref.sub(W, "l0.mix.").items()}
    M["o"] = torch.eye(2, dtype=F64)
    M["norm"][:] = 1.0
    y = torch.randn(1, config["width"], dtype=F64)
    p = (y @ M["in"].T)[0]
    z, xbc, dt = p[:2], ref.silu(p[2:10] * M["conv"][:, 0] + M["conv.b"]), math.log1p(math.exp(float(p[10] + M["dt_bias"][0])))
    x, B, C = xbc[:2], xbc[2:5], xbc[5:]
    out = (dt * (B @ C) + M["D"][0]) * x * ref.silu(z)         # the state before the first token is zero: its decay plays no part
    assert torch.allclose(ref.mixer_mamba2(y, M, config["layers"][0]["mixer"], 1e-5)[0], out / torch.sqrt((out * out).mean() + 1e-5))
