"""Silonex on the layer-list decoder against the float64 restatement (tests/silonex_oracle.py): every mechanism alone, residual streams,
looped blocks, prefill against token-by-token decoding, portions, mixed batches, pages and slots used again, window and page edges in
prompts and in decoding with a key that stands out, a far token that only the recurrent states carry, the first tokens, long decoding,
other sizes, the 16-bit tensor-core attention, greedy generation through the scheduler, the registry and the command line.  All
configurations are made here, small, with random weights exact in bfloat16."""
import importlib
import json
import os
import struct
import subprocess
import sys

import numpy as np
import pytest
import torch

import silonex_oracle as ref

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _models():
    return importlib.import_module("llm-inference-engine_b200.models.silonex")


def _serving():
    return importlib.import_module("llm-inference-engine_b200.serving")


def session(config, packed, dtype="float32", pool_tokens=512, max_seqs=4, max_batch_tokens=512):
    model = _models().SilonexModel(config, packed, dtype=dtype, device=DEV, max_tokens=max_batch_tokens, max_seqs=max_seqs,
                                   max_pages_per_seq=(pool_tokens + 63) // 64)
    return _serving().Session(model, pool_tokens, max_seqs=max_seqs, max_batch_tokens=max_batch_tokens, poison=True)


def tokens_of(config, n, seed):
    return np.random.default_rng(seed).integers(0, config["vocab"], n).tolist()


def replay(sess, requests, schedule):
    """schedule: list of steps, each a list of (name, n) -- the next n tokens of that request, all positions wanted.
    Returns name -> logits [len(tokens), vocab] (numpy)."""
    fed = {k: 0 for k in requests}
    rid, got = {}, {k: [] for k in requests}
    for step in schedule:
        entries, names = [], []
        for name, n in step:
            if name not in rid:
                rid[name] = sess.open()
            toks = requests[name][fed[name]:fed[name] + n]
            assert len(toks) == n
            entries.append((rid[name], toks, list(range(n))))
            names.append((name, n))
            fed[name] += n
        out = sess.feed(entries).cpu().numpy()
        at = 0
        for name, n in names:
            got[name].append(out[at:at + n])
            at += n
        for name, _ in step:
            if fed[name] == len(requests[name]) and name in rid:
                sess.close(rid.pop(name))
    return {k: np.concatenate(v) for k, v in got.items() if v}


def want_logits(config, W, tokens):
    return ref.forward(config, W, tokens).numpy()


def check_all(got, config, W, requests, tol):
    for name, lg in got.items():
        want = want_logits(config, W, requests[name])
        assert not np.isnan(lg).any(), name
        per_pos = np.linalg.norm(lg - want, axis=-1) / np.linalg.norm(want, axis=-1)
        assert per_pos.max() < tol, (name, int(per_pos.argmax()), float(per_pos.max()))


# every mixer, a looped block that starts after the first layer and runs three times, layers with and without a feed-forward
MIXED = [ref.lightning_layer(mlp=ref.dense()), ref.mamba_layer(mlp=ref.dense(24)), ref.pair_layer(window=70),
         ref.mamba_layer(heads=3, vdim=8, state=5, groups=3, conv=2, norm_groups=1), ref.pair_layer(window=9, conv=2, r_heads=2, r_kv_heads=2, mlp=ref.dense()),
         ref.lightning_layer(heads=3, dim=12, vdim=8, decay=[1.0, 0.9, 0.3])]
LOOP = (1, 4, 3)


def _bare_pair():
    """The windowed attention with its window, rotation and cap named null: every key since the start is seen, as it is."""
    layer = ref.pair_layer(heads=2, kv_heads=2, dim=20, vdim=8, r_heads=2, r_kv_heads=1)
    layer["mixer"]["left"].update(mask=None, rot=None, softcap=None)
    return layer


# ------------------------------------------------------------------ each mechanism alone (one-layer models, residual stream compared)
@pytest.mark.parametrize("layer", [
    ref.lightning_layer(),
    ref.lightning_layer(heads=1, dim=5, vdim=3, decay=[0.97]),                                   # nothing a multiple of 4
    ref.lightning_layer(heads=3, dim=80, vdim=40, decay=[0.999, 0.5, 1.0], mlp=ref.dense()),
    ref.lightning_layer(heads=2, dim=136, vdim=12),                                             # key vectors longer than a thread's registers
    ref.mamba_layer(),
    ref.mamba_layer(heads=1, vdim=7, state=3, groups=1, conv=1, norm_groups=1),                  # one head, a convolution of one tap
    ref.mamba_layer(heads=6, vdim=16, state=24, groups=6, conv=4, norm_groups=2, mlp=ref.dense()),  # as many groups as heads
    ref.mamba_layer(heads=4, vdim=5, state=70, groups=1, conv=6, norm_groups=4),                 # norm groups that are whole heads
    ref.mamba_layer(heads=2, vdim=9, state=8, groups=2, conv=2, norm_groups=6),                  # norm groups that cut heads
    ref.pair_layer(),                                                                            # window shorter than a page
    ref.pair_layer(window=100, heads=2, kv_heads=1, dim=24, vdim=40, rot_dims=24, r_heads=4, r_kv_heads=1, r_dim=12, r_vdim=20, conv=4),
    ref.pair_layer(window=1, conv=1, rot_dims=0, scaling=False),                                 # a token sees itself only; no rotation
    ref.pair_layer(window=1000, softcap=0.0, scaling=False, r_heads=1, r_kv_heads=1, r_dim=40, r_vdim=7, conv=6),   # no cap, plain frequencies
    ref.pair_layer(heads=6, kv_heads=6, dim=6, vdim=5, rot_dims=2, base=7.0, softcap=0.7),       # a cap that binds; odd sizes
    ref.pair_layer(window=64, r_heads=2, r_kv_heads=1, r_dim=144, r_vdim=8),
    ref.pair_layer(scaling={"factor": 32.0, "low": 2.0, "high": 3.0, "original": 40}, mlp=ref.dense(7)),
    _bare_pair(),
], ids=["lightning", "lightning_tiny", "lightning_wide", "lightning_long_keys", "mamba", "mamba_tiny", "mamba_groups", "mamba_norm_heads",
        "mamba_norm_cuts", "pair", "pair_sizes", "pair_window_1", "pair_never_binds", "pair_odd", "pair_long_keys", "pair_scaling", "pair_bare"])
@pytest.mark.parametrize("streams", [3, 0], ids=["streams3", "plain"])
def test_one_layer_residual_stream(layer, streams):
    config = ref.make_config([layer], streams=streams)
    W, packed = ref.random_model(config, seed=3)
    toks = tokens_of(config, 150, 1)
    sess = session(config, packed)
    logits, trace = sess.feed([(sess.open(), toks, [0, 1, 149])], trace=True)
    want, res = ref.forward(config, W, toks, trace=True)
    assert ref.rel_err(trace[0].cpu().numpy(), res[0].numpy()) < 3e-5
    assert ref.rel_err(logits.cpu().numpy(), want[[0, 1, 149]].numpy()) < 3e-5


def test_rotation_frequencies_cover_all_three_regimes():
    rot = ref.pair_layer()["mixer"]["left"]["rot"]
    plain = ref.rotary_frequencies({"base": rot["base"], "dims": rot["dims"]})
    ratio = (ref.rotary_frequencies(rot) / plain).tolist()
    assert ratio[0] == 1.0 and ratio[-1] == 1.0 / rot["scaling"]["factor"] and any(1.0 / rot["scaling"]["factor"] < r < 1.0 for r in ratio)


@pytest.mark.parametrize("streams", [1, 2, 5, 8])
def test_stream_counts(streams):
    """One stream with coefficients of its own is not the plain residual sum; eight is the most the engine takes."""
    config = ref.make_config([ref.mamba_layer(mlp=ref.dense()), ref.pair_layer(mlp=ref.dense()), ref.lightning_layer()], streams=streams, logit_scale=1.0)
    W, packed = ref.random_model(config, seed=streams)
    toks = tokens_of(config, 60, 2)
    want, res = ref.forward(config, W, toks, trace=True)
    sess = session(config, packed)
    logits, trace = sess.feed([(sess.open(), toks, list(range(60)))], trace=True)
    for i in range(3):
        assert ref.rel_err(trace[i].cpu().numpy(), res[i].numpy()) < 3e-5, i
    assert ref.rel_err(logits.cpu().numpy(), want.numpy()) < 3e-5


@pytest.mark.parametrize("loop", [None, (0, 1, 1), (0, 2, 2), (1, 3, 3), (2, 3, 2), (0, 3, 2), (1, 2, 0)], ids=str)
def test_looped_blocks_and_constants_that_differ_from_one(loop):
    """Every pass has its own cache and state; nothing else happens between the passes."""
    layers = [ref.lightning_layer(mlp=ref.dense()), ref.pair_layer(window=20), ref.mamba_layer(mlp=ref.dense(8))]
    config = ref.make_config(layers, width=40, vocab=33, loop=loop, logit_scale=1.0)
    W, packed = ref.random_model(config, seed=4)
    toks = tokens_of(config, 90, 2)
    want, res = ref.forward(config, W, toks, trace=True)
    sess = session(config, packed)
    logits, trace = sess.feed([(sess.open(), toks, list(range(90)))], trace=True)
    assert trace.shape[0] == res.shape[0] == 3 + ((loop[1] - loop[0]) * (loop[2] - 1) if loop else 0)
    for i in range(res.shape[0]):
        assert ref.rel_err(trace[i].cpu().numpy(), res[i].numpy()) < 3e-5, i
    assert ref.rel_err(logits.cpu().numpy(), want.numpy()) < 3e-5
    other = dict(config, logit_scale=2.5)   # the constant does something
    sess2 = session(other, packed)
    assert ref.rel_err(sess2.feed([(sess2.open(), toks, list(range(90)))]).cpu().numpy(), 2.5 * want.numpy()) < 3e-5


def test_whole_model_every_layer_fp32_and_bf16():
    config = ref.make_config(MIXED, loop=LOOP)
    W, packed = ref.random_model(config, seed=5)
    toks = tokens_of(config, 200, 3)
    want, res = ref.forward(config, W, toks, trace=True)
    sess = session(config, packed)
    logits, trace = sess.feed([(sess.open(), toks, list(range(200)))], trace=True)
    for i in range(res.shape[0]):
        assert ref.rel_err(trace[i].cpu().numpy(), res[i].numpy()) < 5e-5, i
    assert ref.rel_err(logits.cpu().numpy(), want.numpy()) < 5e-5
    # twelve layer runs whose random stream coefficients enlarge what every run rounds: float16 shows that the 16-bit kernels compute the
    # design, bfloat16 (eight times coarser) stays within eight times that
    for dtype, tol in (("float16", 4e-2), ("bfloat16", 0.3)):
        sess16 = session(config, packed, dtype=dtype)
        logits16, trace16 = sess16.feed([(sess16.open(), toks, list(range(200)))], trace=True)
        assert ref.rel_err(trace16[0].cpu().numpy(), res[0].numpy()) < tol / 20
        assert ref.rel_err(logits16.cpu().numpy(), want.numpy()) < tol


@pytest.mark.parametrize("width,vocab", [(36, 37), (27, 33), (50, 41)], ids=str)
@pytest.mark.parametrize("dtype,tol", [("float32", 3e-5), ("float16", 5e-3), ("bfloat16", 3e-2)], ids=lambda v: str(v))
def test_other_widths_and_vocabularies_in_every_dtype(width, vocab, dtype, tol):
    """Widths and vocabularies that are no multiple of 8 (or of 2), a prompt and decoded tokens, on every engine dtype."""
    layers = [ref.lightning_layer(heads=1, dim=5, vdim=3, decay=[0.97]), ref.mamba_layer(heads=2, vdim=9, state=8, groups=2, conv=2, norm_groups=6),
              ref.mamba_layer(heads=2, vdim=16, state=256, groups=1, conv=4, norm_groups=1), ref.pair_layer(heads=6, kv_heads=6, dim=6, vdim=5, rot_dims=2, base=7.0, softcap=0.7),
              ref.pair_layer(heads=2, kv_heads=1, dim=64, vdim=64, rot_dims=64, window=33, mlp=ref.dense(7))]
    for li, layer in enumerate(layers):
        config = ref.make_config([layer], width=width, vocab=vocab, streams=2)
        W, packed = ref.random_model(config, seed=li)
        toks = tokens_of(config, 100, 1)
        sess = session(config, packed, dtype=dtype)
        r = sess.open()
        got = np.concatenate([sess.feed([(r, toks[:70], list(range(70)))]).cpu().numpy()] + [sess.feed([(r, [t], [0])]).cpu().numpy() for t in toks[70:]])
        assert np.isfinite(got).all() and ref.rel_err(got, want_logits(config, W, toks)) < tol, li


# ------------------------------------------------------------------ schedules
def test_prefill_equals_token_by_token_decoding_and_first_tokens():
    config = ref.make_config(MIXED, loop=LOOP)
    W, packed = ref.random_model(config, seed=6)
    reqs = {"a": tokens_of(config, 80, 4)}
    got = replay(session(config, packed), reqs, [[("a", 1)]] * 80)
    check_all(got, config, W, reqs, 5e-5)
    whole = replay(session(config, packed), reqs, [[("a", 80)]])
    assert ref.rel_err(got["a"], whole["a"]) < 2e-5
    assert ref.rel_err(got["a"][:3], want_logits(config, W, reqs["a"])[:3]) < 3e-5   # the first tokens: empty state, zeros before the convolution


@pytest.mark.parametrize("cuts", [[2] * 60, [1, 2, 3, 5, 8, 13, 21, 34, 33], [63, 1, 1, 55], [64, 6, 50], [69, 2, 49], [7, 113], [23, 1, 24, 2, 70]],
                         ids=lambda c: "-".join(map(str, c[:5])))
def test_portions(cuts):
    config = ref.make_config(MIXED, loop=LOOP)
    W, packed = ref.random_model(config, seed=7)
    reqs = {"a": tokens_of(config, sum(cuts), 5)}
    check_all(replay(session(config, packed), reqs, [[("a", n)] for n in cuts]), config, W, reqs, 1e-4)


def test_long_decoding_lets_windows_pass_over_decoded_tokens_and_pages():
    config = ref.make_config(MIXED, loop=LOOP)
    W, packed = ref.random_model(config, seed=8)
    reqs = {"a": tokens_of(config, 230, 6)}
    check_all(replay(session(config, packed), reqs, [[("a", 10)]] + [[("a", 1)]] * 220), config, W, reqs, 6e-5)


def test_mixed_batches_equal_each_request_alone_and_reuse_pages_and_slots():
    """Six requests over four slots and a pool of six pages: slots and pages are given back and used again while others go on."""
    config = ref.make_config(MIXED, loop=LOOP)
    W, packed = ref.random_model(config, seed=9)
    reqs = {"a": tokens_of(config, 150, 10), "b": tokens_of(config, 9, 11), "c": tokens_of(config, 70, 12), "d": tokens_of(config, 66, 13),
            "e": tokens_of(config, 100, 14), "f": tokens_of(config, 3, 15)}
    schedule = [[("a", 60), ("b", 2), ("c", 1)], [("a", 1), ("b", 7), ("c", 63), ("d", 2)], [("a", 3), ("c", 6), ("d", 64)],
                [("a", 2), ("e", 64)], [("e", 1), ("a", 70), ("f", 3)], [("e", 35), ("a", 14)]]
    sess = session(config, packed, pool_tokens=6 * 64, max_seqs=4, max_batch_tokens=256)
    got = replay(sess, reqs, schedule)
    check_all(got, config, W, reqs, 5e-5)
    assert sess.batcher.free_pages() == 6 and sess.batcher.free_slots() == 4
    for name in reqs:   # and against the same request through a session of its own
        alone = replay(session(config, packed), {name: reqs[name]}, [[(name, len(reqs[name]))]])
        assert ref.rel_err(got[name], alone[name]) < 2e-5, name


@pytest.mark.parametrize("dtype", ["bfloat16", "float16"])
def test_sixteen_bit_logits_do_not_depend_on_the_schedule(dtype):
    config = ref.make_config(MIXED[:4])
    W, packed = ref.random_model(config, seed=10)
    tol = 2e-2 if dtype == "float16" else 0.12
    reqs = {"a": tokens_of(config, 140, 16), "b": tokens_of(config, 30, 17)}
    whole = replay(session(config, packed, dtype=dtype), reqs, [[("a", 140)], [("b", 30)]])
    cut = replay(session(config, packed, dtype=dtype), reqs, [[("a", 64), ("b", 2)], [("a", 9), ("b", 1)], [("a", 2), ("b", 27)], [("a", 65)]])
    for name in reqs:
        want = want_logits(config, W, reqs[name])
        assert ref.rel_err(whole[name], want) < tol and ref.rel_err(cut[name], want) < tol
        assert ref.rel_err(cut[name], whole[name]) < tol


# ------------------------------------------------------------------ edges, with a key that stands out
KEY_TOKEN, QUERY_TOKEN = 7, 11


def _first_layer_input(config, W, token):
    """A first layer's normed input depends on the token alone: every stream holds the embedding output."""
    u = W["embed"][token] * (W["l0.hc1.in"].sum() if config.get("streams") else 1.0)
    return ref.layer_norm(u, W["l0.norm1"], W["l0.norm1.b"], config["norm"]["eps"])


def _bend(W, packed, name, rows, direction, y, gain):
    """Adds gain * direction (over `rows` of the matrix) for the input y, and next to nothing for inputs that are not like y."""
    w = W[name].clone()
    w[rows] += gain * direction[:, None] * (y / (y @ y))[None, :]
    packed[name] = w.to(torch.bfloat16)
    W[name] = packed[name].double()


def _windowed_model(window, seed, dim=32, vdim=12, rot_dims=8, scale=0.3, softcap=30.0):
    """One layer whose sliding-window attention stands alone (the recurrent mixer beside it is weighted by zero: it would carry every
    earlier token past any window).  QUERY_TOKEN's query points at KEY_TOKEN's key, in every head, on the dimensions that do not rotate."""
    config = ref.make_config([ref.pair_layer(heads=2, kv_heads=1, dim=dim, vdim=vdim, window=window, rot_dims=rot_dims, scale=scale, softcap=softcap)])
    W, packed = ref.random_model(config, seed=seed)
    packed["l0.mix.right.out"] = torch.zeros_like(packed["l0.mix.right.out"])
    W["l0.mix.right.out"] = packed["l0.mix.right.out"].double()
    yk, yq = _first_layer_input(config, W, KEY_TOKEN), _first_layer_input(config, W, QUERY_TOKEN)
    key = ref.rms_unit((yk @ W["l0.mix.left.k"].T).view(1, dim), config["norm"]["eps"])[0] * W["l0.mix.left.k.norm"]
    key[:rot_dims] = 0.0
    for h in range(2):
        _bend(W, packed, "l0.mix.left.q", slice(h * dim, (h + 1) * dim), key / (key @ key), yq, 400.0)
    return config, W, packed


def _edge_case(config, W, packed, query_pos, key_pos, seen, decode, dtype="float32", tol=3e-5, pool_tokens=512):
    plain = [t for t in tokens_of(config, 3 * (query_pos + 1), query_pos * 1000 + key_pos) if t not in (KEY_TOKEN, QUERY_TOKEN)][:query_pos + 1]
    with_key, without = list(plain), list(plain)
    with_key[query_pos] = without[query_pos] = QUERY_TOKEN
    if key_pos != query_pos:
        with_key[key_pos] = KEY_TOKEN
    else:   # the query's own position: its own key is always visible; compare with another token's query
        without[query_pos] = plain[query_pos]
    want, want_without = want_logits(config, W, with_key)[query_pos], want_logits(config, W, without)[query_pos]
    changed = ref.rel_err(want_without, want)
    assert changed > 1e-2 if seen else changed == 0.0, changed
    for sequence, expect in ((with_key, want), (without, want_without)):
        sess = session(config, packed, dtype=dtype, pool_tokens=pool_tokens, max_batch_tokens=pool_tokens)
        r = sess.open()
        if decode and query_pos > 0:   # everything before the query is in the pool already; it arrives alone
            sess.feed([(r, sequence[:query_pos], [])])
            got = sess.feed([(r, sequence[query_pos:], [0])]).cpu().numpy()[0]
        else:
            got = sess.feed([(r, sequence, [query_pos])]).cpu().numpy()[0]
        assert ref.rel_err(got, expect) < tol
    return changed


EDGES = [
    (36, 100, 65, True),      # the last key the window keeps: 35 back
    (36, 100, 64, False),     # the first one it has dropped: 36 back
    (36, 35, 0, True),        # the first token of the sequence, just inside
    (36, 36, 0, False),       # ... and just outside
    (36, 37, 1, False), (36, 37, 2, True),
    (64, 127, 64, True), (64, 127, 63, False),     # a window edge that is a page edge
    (64, 128, 64, False), (64, 128, 65, True),
    (100, 150, 63, True), (100, 150, 64, True),    # a page edge inside the window
    (300, 299, 0, True),      # hundreds of keys and four pages back
    (300, 310, 11, True), (300, 310, 10, False),
    (1, 50, 49, False), (1, 50, 50, True),
    (70, 200, 131, True), (70, 200, 130, False),
]


@pytest.mark.parametrize("decode", [False, True], ids=["prompt", "decoded"])
@pytest.mark.parametrize("window,query_pos,key_pos,seen", EDGES, ids=lambda v: str(v))
def test_window_edges_with_a_dominant_key(window, query_pos, key_pos, seen, decode):
    config, W, packed = _windowed_model(window, seed=window + 1)
    _edge_case(config, W, packed, query_pos, key_pos, seen, decode)


@pytest.mark.parametrize("decode", [False, True], ids=["prompt", "decoded"])
@pytest.mark.parametrize("window,query_pos,key_pos,seen", EDGES, ids=lambda v: str(v))
def test_tensor_core_window_edges_with_a_dominant_key(window, query_pos, key_pos, seen, decode):
    config, W, packed = _windowed_model(window, seed=window + 2, dim=64, vdim=32, rot_dims=16, scale=0.25)
    _edge_case(config, W, packed, query_pos, key_pos, seen, decode, dtype="bfloat16", tol=3e-2)


# a window of hundreds of keys over a dozen pages: the per-token kernel takes its widest CTA there, the tiles walk many key blocks
LONG_EDGES = [(600, 700, 101, True), (600, 700, 100, False)]


@pytest.mark.parametrize("decode", [False, True], ids=["prompt", "decoded"])
@pytest.mark.parametrize("window,query_pos,key_pos,seen", LONG_EDGES, ids=lambda v: str(v))
@pytest.mark.parametrize("dtype,tol,sizes", [("float32", 3e-5, {}), ("bfloat16", 3e-2, dict(dim=64, vdim=32, rot_dims=16, scale=0.25))], ids=["fp32", "tiles"])
def test_edges_of_a_window_of_hundreds_of_keys(dtype, tol, sizes, window, query_pos, key_pos, seen, decode):
    config, W, packed = _windowed_model(window, seed=window + 3, **sizes)
    _edge_case(config, W, packed, query_pos, key_pos, seen, decode, dtype=dtype, tol=tol, pool_tokens=768)


def _far_model(kind, seed):
    """One recurrent layer in which KEY_TOKEN writes a large key and QUERY_TOKEN reads along it: hundreds of tokens later the write
    shows, if the state was carried all the way."""
    if kind == "lightning":
        config = ref.make_config([ref.lightning_layer(heads=2, dim=8, vdim=12, decay=[1.0, 0.998])])
        W, packed = ref.random_model(config, seed=seed)
        direction = torch.ones(16, dtype=torch.float64)
        kname, qname, rows = "l0.mix.k", "l0.mix.q", slice(0, 16)
    else:
        config = ref.make_config([ref.mamba_layer(heads=2, vdim=6, state=8, groups=1, conv=1, norm_groups=1)])
        W, packed = ref.random_model(config, seed=seed)
        packed["l0.mix.A_log"] = torch.full_like(packed["l0.mix.A_log"], -9.0)   # decay exp(-exp(-9) dt): next to 1
        packed["l0.mix.conv"] = torch.ones_like(packed["l0.mix.conv"])
        packed["l0.mix.conv.b"] = torch.zeros_like(packed["l0.mix.conv.b"])
        for n in ("A_log", "conv", "conv.b"):
            W["l0.mix." + n] = packed["l0.mix." + n].double()
        direction = torch.ones(8, dtype=torch.float64)
        inner = 12
        kname = qname = "l0.mix.in"
        rows = None
    yk, yq = _first_layer_input(config, W, KEY_TOKEN), _first_layer_input(config, W, QUERY_TOKEN)
    if rows is not None:
        _bend(W, packed, kname, rows, direction, yk, 30.0)
        _bend(W, packed, qname, rows, direction, yq, 30.0)
    else:   # rows z | x | B | C | dt
        _bend(W, packed, kname, slice(2 * inner, 2 * inner + 8), direction, yk, 30.0)
        _bend(W, packed, qname, slice(2 * inner + 8, 2 * inner + 16), direction, yq, 30.0)
    return config, W, packed


@pytest.mark.parametrize("decode", [False, True], ids=["prompt", "decoded"])
@pytest.mark.parametrize("query_pos,key_pos", [(310, 0), (310, 1), (400, 63), (400, 64), (255, 128), (5, 0)], ids=str)
@pytest.mark.parametrize("kind", ["lightning", "mamba2"])
def test_far_tokens_that_only_the_state_carries(kind, query_pos, key_pos, decode):
    config, W, packed = _far_model(kind, seed=query_pos)
    _edge_case(config, W, packed, query_pos, key_pos, True, decode, tol=5e-5)


# ------------------------------------------------------------------ the tensor-core attention of 16-bit engines
@pytest.mark.parametrize("dtype", ["bfloat16", "float16"])
@pytest.mark.parametrize("dim,vdim", [(32, 32), (64, 128), (128, 64), (64, 32)])
def test_tensor_core_attention_against_the_oracle_and_against_single_tokens(dim, vdim, dtype):
    """Portions of eight tokens and more take the tensor-core kernel, shorter ones the per-token kernel: both against the oracle, and
    against each other on the same sequence; one layer's cap binds, the other's does not."""
    layers = [ref.pair_layer(heads=4, kv_heads=2, dim=dim, vdim=vdim, rot_dims=dim // 2, window=50, softcap=2.0, scale=0.5, mlp=ref.dense()),
              ref.pair_layer(heads=2, kv_heads=2, dim=dim, vdim=vdim, rot_dims=dim, window=90, softcap=0.0, scale=dim ** -0.5, mlp=ref.dense())]
    config = ref.make_config(layers, width=64)
    W, packed = ref.random_model(config, seed=dim + vdim)
    reqs = {"a": tokens_of(config, 200, 20)}
    want = want_logits(config, W, reqs["a"])
    tiles = replay(session(config, packed, dtype=dtype), reqs, [[("a", 130)], [("a", 70)]])["a"]
    single = replay(session(config, packed, dtype=dtype), reqs, [[("a", 7)]] * 28 + [[("a", 4)]])["a"]
    assert ref.rel_err(tiles, want) < 4e-2 and ref.rel_err(single, want) < 4e-2 and ref.rel_err(tiles, single) < 3e-2


# ------------------------------------------------------------------ the recurrence's launcher alone
@pytest.mark.parametrize("heads,kv_heads,dim,vdim", [(4, 2, 16, 12), (3, 3, 7, 5), (2, 1, 136, 20), (8, 8, 64, 64)], ids=str)
def test_decay_recurrence_launcher_against_a_plain_loop(heads, kv_heads, dim, vdim):
    """Three sequences in one call: one from position 0 (its slot's old state must not show), one that continues from its slot's state, a
    single token; fp32 against a float64 loop."""
    import ctypes as C

    m = importlib.import_module("llm-inference-engine_b200")
    pad4 = lambda n: (n + 3) & ~3
    q0, k0 = 0, pad4(kv_heads * dim)
    v0 = k0 + pad4(kv_heads * dim)
    s0 = v0 + pad4(heads * vdim)
    d0 = s0 + pad4(heads * vdim)
    ld = d0 + pad4(heads)
    gen = torch.Generator().manual_seed(dim)
    lens, pos0, slots = [37, 20, 1], [0, 5, 9], [2, 0, 1]
    T = sum(lens)
    rec = torch.randn(T, ld, generator=gen)
    rec[:, d0:d0 + heads] = 0.5 + 0.5 * torch.rand(T, heads, generator=gen)
    rec[3, d0] = 1.0
    state = torch.randn(3, heads, dim, vdim, generator=gen)
    want_o, want_state = torch.zeros(T, heads * vdim, dtype=torch.float64), state.double().clone()
    t = 0
    for n, p, slot in zip(lens, pos0, slots):
        S = torch.zeros(heads, dim, vdim, dtype=torch.float64) if p == 0 else state[slot].double().clone()
        for _ in range(n):
            r = rec[t].double()
            for h in range(heads):
                g = h // (heads // kv_heads)
                S[h] = r[d0 + h] * S[h] + torch.outer(r[k0 + g * dim:k0 + (g + 1) * dim], r[v0 + h * vdim:v0 + (h + 1) * vdim])
                want_o[t, h * vdim:(h + 1) * vdim] = S[h].T @ r[q0 + g * dim:q0 + (g + 1) * dim]
            t += 1
        want_state[slot] = S
    d_rec, d_state, d_o = rec.to(DEV), state.to(DEV), torch.full((T, heads * vdim), float("nan"), device=DEV)
    ints = [torch.tensor(a, dtype=torch.int32, device=DEV) for a in ([0, 37, 57, 58], pos0, slots)]
    m.check(m.lib().b200_decay_recurrent(m.ptr(d_rec), m.ptr(d_state), m.ptr(d_o), m.ptr(ints[0]), m.ptr(ints[1]), m.ptr(ints[2]), 3, heads, kv_heads,
                                          dim, vdim, m.stream()))
    assert ref.rel_err(d_o.cpu(), want_o) < 1e-5 and ref.rel_err(d_state.cpu(), want_state) < 1e-5


# ------------------------------------------------------------------ state that is carried, and state that must not be
def test_a_slot_used_again_starts_from_nothing():
    """The second request takes the slot and the pages of the first: neither its matrix states nor the convolutions' inputs may show."""
    config = ref.make_config(MIXED, loop=LOOP)
    W, packed = ref.random_model(config, seed=11)
    reqs = {"a": tokens_of(config, 70, 21), "b": tokens_of(config, 40, 22)}
    sess = session(config, packed, pool_tokens=128, max_seqs=1, max_batch_tokens=128)
    got = replay(sess, reqs, [[("a", 70)], [("b", 1)], [("b", 2)], [("b", 37)]])
    check_all(got, config, W, reqs, 5e-5)


def test_convolution_inputs_are_carried_across_portions_shorter_than_the_taps():
    config = ref.make_config([ref.pair_layer(conv=6, window=5), ref.mamba_layer(conv=5)])
    W, packed = ref.random_model(config, seed=12)
    reqs = {"a": tokens_of(config, 30, 23)}
    check_all(replay(session(config, packed), reqs, [[("a", n)] for n in (1, 1, 2, 1, 3, 1, 1, 7, 2, 11)]), config, W, reqs, 3e-5)


def test_pool_exhaustion_is_refused_not_overwritten():
    config = ref.make_config(MIXED[:3])
    W, packed = ref.random_model(config, seed=13)
    sess = session(config, packed, pool_tokens=128, max_seqs=2, max_batch_tokens=256)
    a, b = sess.open(), sess.open()
    sess.feed([(a, tokens_of(config, 100, 1), [])])
    with pytest.raises(Exception):
        sess.feed([(b, tokens_of(config, 10, 2), [])])   # a has both pages


def test_more_streams_than_the_engine_takes_are_refused():
    config = ref.make_config([ref.lightning_layer()], streams=9)
    W, packed = ref.random_model(config, seed=14)
    with pytest.raises(Exception):
        session(config, packed)


# ------------------------------------------------------------------ the scheduler's own entry point, the registry, the command line
@pytest.mark.parametrize("chunk", [0, 5])
def test_greedy_generation_through_the_scheduler(chunk):
    config = ref.make_config(MIXED, loop=LOOP)
    W, packed = ref.random_model(config, seed=30)
    prompts = [tokens_of(config, n, 40 + n) for n in (1, 9, 70, 23, 2, 65)]   # six requests over four slots
    sess = session(config, packed, pool_tokens=6 * 64, max_seqs=4, max_batch_tokens=128)
    out = sess.generate(prompts, 10, chunk=chunk)
    for p, ids in zip(prompts, out):
        assert ids == ref.greedy(config, W, p, 10)
    assert sess.batcher.free_pages() == 6 and sess.batcher.free_slots() == 4


def _write_checkpoint(folder, config, packed):
    header, blob = {}, b""
    for k, v in packed.items():
        raw = v.contiguous().view(torch.int16).numpy().tobytes()
        header[k] = {"dtype": "BF16", "shape": list(v.shape), "data_offsets": [len(blob), len(blob) + len(raw)]}
        blob += raw
    hj = json.dumps(header).encode()
    (folder / "model.safetensors").write_bytes(struct.pack("<Q", len(hj)) + hj + blob)
    (folder / "config.json").write_text(json.dumps(config))


def test_registry_loads_a_checkpoint_folder(tmp_path):
    config = ref.make_config(MIXED[:3], loop=(0, 2, 2))
    W, packed = ref.random_model(config, seed=33)
    _write_checkpoint(tmp_path, config, packed)
    model = importlib.import_module("llm-inference-engine_b200.models").load_model(str(tmp_path), dtype="float32", device=DEV, max_tokens=128, max_seqs=2)
    sess = _serving().Session(model, 128, max_seqs=2)
    toks = tokens_of(config, 20, 1)
    got = sess.feed([(sess.open(), toks, [19])]).cpu().numpy()
    assert ref.rel_err(got, want_logits(config, W, toks)[[19]]) < 5e-5


def test_trace_command_line_replays_a_schedule(tmp_path):
    config = ref.make_config(MIXED, loop=LOOP)
    W, packed = ref.random_model(config, seed=34)
    _write_checkpoint(tmp_path, config, packed)
    a, b = tokens_of(config, 80, 1), tokens_of(config, 5, 2)
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": a[:70], "want": [0, 69]}], "end": []},
             {"step": 1, "entries": [{"id": "a", "tokens": a[70:72], "want": []}, {"id": "b", "tokens": b[:4], "want": [3]}], "end": []},
             {"step": 2, "entries": [{"id": "b", "tokens": b[4:], "want": [0]}, {"id": "a", "tokens": a[72:], "want": [7]}], "end": ["a", "b"]}]
    out = tmp_path / "out"
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", str(tmp_path), "--dtype", "float32", "--out", str(out),
                        "--max-tokens", "192"], input="".join(json.dumps(s) + "\n" for s in steps), capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    assert [l for l in r.stdout.splitlines() if l.startswith("done")] == ["done 0", "done 1", "done 2"]
    wa, wb = want_logits(config, W, a), want_logits(config, W, b)
    got0 = np.fromfile(out / "0.f32", dtype="<f4").reshape(2, -1)
    got1 = np.fromfile(out / "1.f32", dtype="<f4").reshape(1, -1)
    got2 = np.fromfile(out / "2.f32", dtype="<f4").reshape(2, -1)
    assert ref.rel_err(got0, wa[[0, 69]]) < 5e-5 and ref.rel_err(got1, wb[[3]]) < 5e-5 and ref.rel_err(got2, np.stack([wb[4], wa[79]])) < 5e-5
