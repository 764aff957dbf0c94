"""Host-side checks of the Fedovik model class (no GPU): the registry, the configuration reader, and the oracle's own mechanisms."""
import importlib

import pytest
import torch

import fedovik_oracle as ref
from util import b200


def test_registry_names_the_design():
    models = importlib.import_module("llm-inference-engine_b200.models")
    assert "fedovik" in models.architectures()
    assert models.architecture_of({"architecture": "Fedovik"}) == "Fedovik"


def test_layer_specs_follow_the_configuration():
    m = b200()
    f = importlib.import_module("llm-inference-engine_b200.models.fedovik")
    config = ref.make_config([ref.attention_layer(heads=6, kv_heads=3, dim=10, vdim=7, rot_dims=4, base=77.0, scale=0.5, mlp=ref.dense(13)),
                              ref.pair_layer(heads=4, kv_heads=1, dim=12, vdim=20, window=11, scale=0.3, left_scale=0.6, right_scale=1.4, r_heads=6,
                                             r_kv_heads=2, r_dim=5, r_vdim=9, conv=3),
                              ref.mlstm_layer(heads=3, dim=8, vdim=14, gate_cap=9.0)])
    a, b, c = f.layer_specs(config)
    assert (a["mixer"], a["norm"], a["heads"], a["kv_heads"], a["dim"], a["vdim"], a["rot_dims"], a["window"], a["attn_weight"], a["out_gate"]) == \
        (m.MIXER_ATTN_SCORED, m.NORM_LN_PARALLEL, 6, 3, 10, 7, 4, 0, m.ATTN_SIGMOID, 1)
    assert a["scale"] == 0.5 and a["rot_base"] == 77.0 and (a["mlp"], a["expert_ff"], a["act"], a["gated"]) == (m.MLP_DENSE, 13, m.ACT_RELU, 1)
    assert (b["mixer"], b["heads"], b["kv_heads"], b["dim"], b["vdim"], b["window"], b["rot_dims"], b["attn_weight"], b["out_gate"], b["mlp"]) == \
        (m.MIXER_ATTN_SCORED, 4, 1, 12, 20, 11, 0, m.ATTN_SOFTMAX, 0, m.MLP_NONE)
    assert b["scale"] == 0.3 and b["mix_scale"] == 0.6 and b["side_scale"] == 1.4
    s = b["side"]
    assert (s["mixer"], s["heads"], s["kv_heads"], s["dim"], s["vdim"], s["conv"]) == (m.MIXER_DELTA, 6, 2, 5, 9, 3)
    assert (c["mixer"], c["heads"], c["dim"], c["vdim"], c["gate_cap"], c["mlp"]) == (m.MIXER_MLSTM, 3, 8, 14, 9.0, m.MLP_NONE)
    with pytest.raises(ValueError):
        f.layer_specs(ref.make_config([{"type": "conv", "mixer": {"heads": 1, "dim": 4}, "mlp": None}]))
    with pytest.raises(ValueError):
        f.layer_specs(ref.make_config([ref.mlstm_layer(mlp={"kind": "moe"})]))


def test_oracle_run_order_of_looped_blocks():
    assert ref.layer_order(ref.make_config([0] * 4)) == [(0, None), (1, None), (2, None), (3, None)]
    assert ref.layer_order(ref.make_config([0] * 4, loop=(1, 3, 2))) == [(0, None), (1, 0), (2, None), (1, 1), (2, None), (3, None)]
    assert ref.layer_order(ref.make_config([0] * 2, loop=(0, 1, 1))) == [(0, 0), (1, None)]


def test_oracle_rotation_pairs_neighbours_and_leaves_the_rest():
    v = (torch.arange(12, dtype=torch.float64) + 1).view(2, 1, 6)
    out = ref.rotate_interleaved(v, torch.tensor([0, 3]), 4, 100.0)
    assert torch.equal(out[0], v[0])                         # position 0 turns nothing
    assert torch.equal(out[1, 0, 4:], v[1, 0, 4:])           # past `dims`: unchanged
    c, s = torch.cos(torch.tensor(3.0, dtype=torch.float64)), torch.sin(torch.tensor(3.0, dtype=torch.float64))
    assert torch.allclose(out[1, 0, 0], v[1, 0, 0] * c - v[1, 0, 1] * s) and torch.allclose(out[1, 0, 1], v[1, 0, 1] * c + v[1, 0, 0] * s)
    c2, s2 = torch.cos(torch.tensor(0.3, dtype=torch.float64)), torch.sin(torch.tensor(0.3, dtype=torch.float64))   # 3 * 100^(-2/4)
    assert torch.allclose(out[1, 0, 2], v[1, 0, 2] * c2 - v[1, 0, 3] * s2)


def test_oracle_convolution_is_causal_and_ends_on_the_current_token():
    z = torch.randn(7, 2, dtype=torch.float64)
    taps = torch.tensor([[0.0, 0.0, 1.0], [1.0, 0.0, 0.0]], dtype=torch.float64)
    out = ref.short_conv_silu(z, taps)
    silu = lambda t: t * torch.sigmoid(t)
    assert torch.allclose(out[:, 0], silu(z[:, 0]))                                       # the last tap alone: the token itself
    assert torch.allclose(out[2:, 1], silu(z[:-2, 1])) and torch.equal(out[:2, 1], torch.zeros(2, dtype=torch.float64))


def test_oracle_delta_rule_writes_before_it_reads():
    """With no decay, a full step and a unit key, the token's own value comes straight back."""
    config = ref.make_config([ref.pair_layer(r_heads=1, r_kv_heads=1, r_dim=4, r_vdim=3, conv=1)])
    W, _ = ref.make_weights(config, seed=1)
    mx = config["layers"][0]["mixer"]["right"]
    R = {k[len("l0.mix.right."):]: v.clone() for k, v in W.items() if k.startswith("l0.mix.right.")}
    R["A_log"][:] = -60.0                      # decay exp(-tiny) = 1
    R["b"][:] = 0.0
    R["b"] += 1e3 * torch.ones_like(R["b"])    # beta -> 1 for inputs of positive sum; use a fixed positive input below
    y = torch.ones(1, config["width"], dtype=torch.float64)
    q = ref.short_conv_silu(y @ R["q"].T, R["q.conv"])
    k = ref.short_conv_silu(y @ R["k"].T, R["k.conv"])
    v = ref.short_conv_silu(y @ R["v"].T, R["v.conv"])
    qn, kn = q / torch.sqrt((q * q).sum() + 1e-6) * 4 ** -0.5, k / torch.sqrt((k * k).sum() + 1e-6)
    R["norm"][:] = 1.0
    R["g2"][:] = 0.0                           # gate sigmoid(0) = 1/2
    R["o"] = torch.eye(3, dtype=torch.float64)
    out = ref.mixer_gated_delta(y, R, mx, 0.0)
    o = (kn @ qn.T) * v                        # S = k v^T after one token
    assert torch.allclose(out, 0.5 * o / torch.sqrt((o * o).mean()), atol=1e-9)


def test_oracle_matrix_memory_starts_its_maximum_at_zero():
    """A very negative input gate on the first token: the running maximum stays 0 + f, it does not drop to the gate."""
    config = ref.make_config([ref.mlstm_layer(heads=1, dim=2, vdim=2, gate_cap=50.0)])
    W, _ = ref.make_weights(config, seed=2)
    M = {k[len("l0.mix."):]: v.clone() for k, v in W.items() if k.startswith("l0.mix.")}
    M["i"][:] = 0.0
    M["i.b"][:] = -30.0
    M["f"][:] = 0.0
    M["f.b"][:] = 40.0                           # log forget gate ~ 0
    M["g"][:] = 0.0
    M["norm"][:] = 1.0
    M["o"] = torch.eye(2, dtype=torch.float64)
    y = torch.randn(1, config["width"], dtype=torch.float64)
    q, k, v = (y @ M["q"].T)[0] * 2 ** -0.5, (y @ M["k"].T)[0], (y @ M["v"].T)[0]
    b = torch.exp(50.0 * torch.tanh(torch.tensor(-30.0 / 50.0, dtype=torch.float64)))      # exp(i - m) with m = 0, i soft-capped
    o = b * (k @ q) * v / (torch.maximum((b * (k @ q)).abs(), torch.tensor(1.0, dtype=torch.float64)) + 1e-6)
    want = 0.5 * o / torch.sqrt((o * o).mean() + 1e-5)
    assert torch.allclose(ref.mixer_mlstm(y, M, config["layers"][0]["mixer"], 1e-5), want[None], rtol=1e-6, atol=1e-12)
