"""The slow Tudatar implementation of tests/tudatar_oracle.py against itself and against hand-made cases (no GPU):
whole-sequence arithmetic == the same fed in portions, and each mechanism on inputs whose answer is known in closed form.
The model-folder writer is checked against a byte-level read of its own file."""
import json
import math
import struct

import numpy as np

import tudatar_oracle as O


def small_cfg():
    return O.make_config([
        O.latent_layer(),
        O.window_layer(window=5),
        O.delta_layer(conv=3),
        O.window_layer(heads=2, kv_heads=2, window=40, mlp=None),
        O.delta_layer(heads=2, kv_heads=1, dim=8, vdim=8, conv=1, mlp=O.moe(experts=3, top=3)),
    ], width=24, vocab=37)


def test_whole_sequence_equals_portions_and_single_tokens():
    cfg = small_cfg()
    W = O.random_weights(cfg, seed=3)
    toks = np.random.default_rng(0).integers(0, cfg["vocab"], 19).tolist()
    whole, outs = O.forward(cfg, W, toks)
    assert outs.shape == (5, 19, 24)
    for cuts in ([1] * 19, [2, 3, 5, 7, 2], [18, 1]):
        inc, got, at = O.StepOracle(cfg, W), [], 0
        for c in cuts:
            got.append(inc.step(toks[at:at + c])[0])
            at += c
        assert np.allclose(np.concatenate(got), whole, rtol=0, atol=1e-9)


def test_tanh_norm_uses_no_statistics():
    W = {"n": np.array([2.0, 3.0]), "n.b": np.array([0.5, -0.5]), "n.alpha": np.array(0.25)}
    x = np.array([[4.0, -8.0], [400.0, 0.0]])
    got = O.tanh_norm(x, W, "n")
    assert np.allclose(got[0], [2 * math.tanh(1.0) + 0.5, 3 * math.tanh(-2.0) - 0.5])
    assert np.allclose(got[1], [2.5, -0.5])   # saturates; a zero input gives the shift alone


def test_rotation_pairs_neighbours_and_rescales_slow_frequencies():
    rot = {"base": 100.0, "dims": 4}
    f, mult = O.rot_freqs(rot)
    assert np.allclose(f, [1.0, 0.1]) and mult == 1.0
    z = np.arange(1.0, 7.0).reshape(1, 6)
    r = O.rotate_pairs(z, [3], rot)
    a0, a1 = 3.0, 0.3
    assert np.allclose(r[0], [1 * math.cos(a0) - 2 * math.sin(a0), 2 * math.cos(a0) + 1 * math.sin(a0),
                              3 * math.cos(a1) - 4 * math.sin(a1), 4 * math.cos(a1) + 3 * math.sin(a1), 5, 6])
    assert np.allclose(O.rotate_pairs(z, [0], rot), z)
    # rescaling: 16 dims, base 10000, original length 64; fast = 8 turns, slow = 1 turn
    rot = {"base": 10000.0, "dims": 16, "scaling": {"factor": 4.0, "fast": 8.0, "slow": 1.0, "original": 64}}
    f0 = np.array([10000.0 ** (-2.0 * i / 16) for i in range(8)])
    lo = math.floor(16 * math.log(64 / (2 * math.pi * 8)) / (2 * math.log(10000.0)))
    hi = math.ceil(16 * math.log(64 / (2 * math.pi * 1)) / (2 * math.log(10000.0)))
    assert (lo, hi) == (0, 3)
    f, mult = O.rot_freqs(rot)
    assert math.isclose(mult, 0.1 * math.log(4.0) + 1.0)
    assert np.allclose(f[0], f0[0]) and np.allclose(f[3:], f0[3:] / 4.0)   # fast pairs untouched, slow pairs slowed down
    assert np.allclose(f[1], f0[1] / 4.0 * (1 / 3) + f0[1] * (2 / 3))
    # cos and sin carry the multiplier: a rotated pair's length grows by it
    v = O.rotate_pairs(np.array([[1.0, 0.0] + [0.0] * 14]), [5], rot)
    assert math.isclose(math.hypot(v[0, 0], v[0, 1]), mult)


def test_causal_conv_continues_from_its_tail():
    w = np.array([[1.0, 10.0, 100.0], [0.5, 0.0, 2.0]])   # last column: the current token
    x = np.arange(1.0, 11.0).reshape(5, 2)
    y, tail = O.causal_conv(x, w, np.zeros((2, 2)))
    assert np.allclose(y[0], [100.0 * 1, 2.0 * 2]) and np.allclose(y[2], [1 * 1 + 10 * 3 + 100 * 5, 0.5 * 2 + 2 * 6])
    assert np.allclose(tail, x[3:])
    y1, t1 = O.causal_conv(x[:2], w, np.zeros((2, 2)))
    y2, t2 = O.causal_conv(x[2:], w, t1)
    assert np.allclose(np.concatenate([y1, y2]), y) and np.allclose(t2, tail)
    y3, t3 = O.causal_conv(x, w[:, 2:], np.zeros((0, 2)))   # one tap: no memory
    assert np.allclose(y3, x * w[:, 2]) and t3.shape == (0, 2)


def test_delta_rule_writes_then_reads_and_decays_per_channel():
    # one head, two key channels, one value channel; unit keys along the axes
    k = np.array([[[1.0, 0.0]], [[0.0, 1.0]], [[1.0, 0.0]]])
    q = k.copy()
    v = np.array([[[5.0]], [[7.0]], [[1.0]]])
    g = np.ones((3, 1, 2))
    beta = np.ones((3, 1))
    S = np.zeros((1, 2, 1))
    o = O.delta_scan(q, k, v, g, beta, S)
    # beta = 1 replaces what the key holds; the read-out sees the write of its own token
    assert np.allclose(o[:, 0, 0], [5.0, 7.0, 1.0]) and np.allclose(S[0, :, 0], [1.0, 7.0])
    # decay acts on the key channel's row before the token's write, and only on that row
    S = np.array([[[4.0], [8.0]]])
    g = np.array([[[0.5, 1.0]]])
    o = O.delta_scan(np.array([[[1.0, 1.0]]]), np.array([[[0.0, 0.0]]]), np.array([[[0.0]]]), g, np.ones((1, 1)), S)
    assert np.allclose(S[0, :, 0], [2.0, 8.0]) and np.allclose(o[0, 0, 0], 10.0)
    # beta = 0.5 moves the stored value half way
    S = np.array([[[4.0], [0.0]]])
    O.delta_scan(q[:1], k[:1], np.array([[[10.0]]]), np.ones((1, 1, 2)), np.array([[0.5]]), S)
    assert np.allclose(S[0, 0, 0], 7.0)


def test_window_and_distance_penalty():
    """one head, identical keys and a zero query: the weights are softmax(-r1 ln(1 + r2 d)) over the window"""
    cfg = O.make_config([O.window_layer(heads=1, kv_heads=1, dim=4, vdim=4, window=3, mlp=None)], width=4, vocab=5)
    W = O.random_weights(cfg, seed=1)
    W["l0.mix.q"][:] = 0.0
    W["l0.mix.q.b"][:] = 0.0
    W["l0.mix.r1"][:] = 2.0
    W["l0.mix.r2"][:] = 0.5
    W["l0.mix.o"] = np.eye(4)
    h = np.random.default_rng(0).standard_normal((6, 4))
    st = {}
    y = O.window_mixer(h, W, "l0.mix.", cfg["layers"][0]["mixer"], 1e-5, st, 0)
    v = st["v"][:, 0]
    assert np.allclose(np.sqrt((v * v).mean(-1)), 1.0, atol=1e-4)   # values are cached with unit root mean square
    w = np.array([(1 + 0.5 * d) ** -2.0 for d in range(3)])
    assert np.allclose(y[5], (w[0] * v[5] + w[1] * v[4] + w[2] * v[3]) / w.sum())   # position 2 is outside the window of 3
    assert np.allclose(y[1], (w[0] * v[1] + w[1] * v[0]) / w[:2].sum())
    assert np.allclose(y[0], v[0])


def test_joint_norm_runs_over_all_heads_at_once():
    cfg = O.make_config([O.window_layer(heads=2, kv_heads=2, dim=2, vdim=2, window=8, mlp=None)], width=4, vocab=5)
    W = O.random_weights(cfg, seed=2)
    W["l0.mix.k"] = np.eye(4)
    W["l0.mix.k.b"] = np.array([1.0, 0.0, 0.0, 0.0])
    W["l0.mix.k.norm"] = np.array([1.0, 1.0, 1.0, 2.0])
    st = {}
    O.window_mixer(np.array([[2.0, 0.0, 0.0, 4.0]]), W, "l0.mix.", cfg["layers"][0]["mixer"], 0.0, st, 0)
    r = math.sqrt((9.0 + 16.0) / 4.0)
    assert np.allclose(st["k"].reshape(4), [3.0 / r, 0.0, 0.0, 8.0 / r])   # per head it would be 3/sqrt(4.5) and 8/sqrt(8)


def test_latent_attention_caches_one_latent_and_one_rotated_part():
    cfg = O.make_config([O.latent_layer(heads=2, dim=4, rot_dim=4, vdim=6, kv_rank=5, q_rank=7, mlp=None)], width=8, vocab=5)
    W = O.random_weights(cfg, seed=3)
    h = np.random.default_rng(1).standard_normal((4, 8))
    m = cfg["layers"][0]["mixer"]
    st = {}
    y = O.latent_mixer(h, W, "l0.mix.", m, 1e-5, st, 0)
    assert st["c"].shape == (4, 5) and st["kr"].shape == (4, 4)
    # the same through explicit per-head keys and values, token 3 only
    c = O.rms((h @ W["l0.mix.dkv"].T)[:, :5], 1e-5) * W["l0.mix.dkv.norm"]
    assert np.allclose(c, st["c"])
    kr = O.rotate_pairs((h @ W["l0.mix.dkv"].T)[:, 5:], range(4), m["rot"])
    q = ((O.rms(h @ W["l0.mix.dq"].T, 1e-5) * W["l0.mix.dq.norm"]) @ W["l0.mix.uq"].T).reshape(4, 2, 8)
    out = []
    for hd in range(2):
        k = np.concatenate([c @ W["l0.mix.uk"][hd * 4:(hd + 1) * 4].T, kr], 1)
        qq = np.concatenate([q[3, hd, :4], O.rotate_pairs(q[3:4, hd, 4:], [3], m["rot"])[0]])
        s = k @ qq * m["scale"]
        a = np.exp(s - s.max())
        out.append((a / a.sum()) @ (c @ W["l0.mix.uv"][hd * 6:(hd + 1) * 6].T))
    assert np.allclose(y[3], np.concatenate(out) @ W["l0.mix.o"].T)


def test_router_chooses_with_the_correction_and_weighs_without_it():
    r = {"experts": 4, "top": 2, "scale": 3.0}
    W = {"p.router": np.eye(4)[:, :4], "p.correction": np.array([0.0, 0.0, 0.0, 10.0])}
    h = np.array([[2.0, 1.0, 0.0, -5.0]])
    idx, w = O.route(h, W, "p.", r)
    s = 1.0 / (1.0 + np.exp(-h[0]))
    assert idx[0].tolist() == [3, 0]   # expert 3 wins through its correction only
    assert np.allclose(w[0], np.array([s[3], s[0]]) / (s[3] + s[0]) * 3.0)
    assert math.isclose(w.sum(), 3.0)


def test_write_model_layout(tmp_path):
    cfg = small_cfg()
    W = O.random_weights(cfg, seed=4)
    d = O.write_model(str(tmp_path / "m"), cfg, W)
    raw = open(d + "/model.safetensors", "rb").read()
    n = struct.unpack("<Q", raw[:8])[0]
    hdr = json.loads(raw[8:8 + n])
    assert n % 8 == 0 and set(hdr) == set(W)
    e = hdr["l2.mix.q.conv"]
    assert e["dtype"] == "BF16" and e["shape"] == [24, 3]
    bits = np.frombuffer(raw[8 + n + e["data_offsets"][0]:8 + n + e["data_offsets"][1]], np.uint16)
    assert np.array_equal((bits.astype(np.uint32) << 16).view(np.float32).reshape(24, 3), W["l2.mix.q.conv"].astype(np.float32))
    assert hdr["final.norm.alpha"]["shape"] == []
    assert json.load(open(d + "/config.json"))["layers"][0]["type"] == "latent_attention"


def test_the_packaged_writer_names_the_same_tensors():
    """lmrs_b200.model_dir (random models for benchmarks) and this file's table agree on names and shapes"""
    from lmrs_b200 import model_dir as md
    cfg = md.tudatar_config(48, 5, 90, heads=4, kv_heads=2, head_dim=8, window=12, delta_heads=3, delta_dim=16, conv=3, kv_rank=20,
                            q_rank=28, rot_dim=6, experts=5, top=2, expert_ff=24, low_rank=6)
    assert [L["type"] for L in cfg["layers"]] == ["channel_delta", "attention", "channel_delta", "latent_attention", "channel_delta"]
    a = {n: tuple(s) for n, s, _ in md.tudatar_tensors(cfg)}
    b = {n: tuple(s) for n, s, _ in O.tensor_table(cfg)}
    assert a == b
    # the chosen experts' share of the expert matrices, everything else once
    dense = sum(int(np.prod(s)) for n, s in a.items() if ".mlp.e" not in n and n != "embed")
    experts = sum(int(np.prod(s)) for n, s in a.items() if ".mlp.e" in n)
    assert md.tudatar_param_bytes(cfg) == int((dense + a["embed"][1] + experts * 2 / 5) * 2)
    W = O.random_weights(cfg, seed=1)
    logits, _ = O.forward(cfg, W, [1, 2, 3])
    assert logits.shape == (3, 90) and np.isfinite(logits).all()
